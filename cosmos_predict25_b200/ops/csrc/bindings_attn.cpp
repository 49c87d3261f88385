// Attention operators of torch.ops.cosmos_b200.

#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include <tuple>

#include "launchers.h"

int* cb200_error_word(int device);

namespace {
using at::Tensor;

inline void check_qkv(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kBFloat16 && t.is_contiguous() && t.dim() == 4 && t.size(3) == 128, name,
              " must be a contiguous CUDA bf16 tensor [B, S, H, 128]");
}

// q [B,Sq,H,128], k/v [B,Skv,H,128] -> (o [B,Sq,H,128], lse [B,H,Sq] fp32, natural log)
std::tuple<Tensor, Tensor> fa_fwd_variant(const Tensor& q, const Tensor& k, const Tensor& v, double scale, int64_t variant) {
  check_qkv(q, "q");
  check_qkv(k, "k");
  check_qkv(v, "v");
  TORCH_CHECK(k.sizes() == v.sizes() && q.size(0) == k.size(0) && q.size(2) == k.size(2), "q/k/v shape mismatch");
  c10::cuda::CUDAGuard g(q.device());
  const int B = (int)q.size(0), Sq = (int)q.size(1), H = (int)q.size(2), Skv = (int)k.size(1);
  Tensor o = at::empty_like(q);
  Tensor lse = at::empty({B, H, Sq}, q.options().dtype(at::kFloat));
  const int rc = cb200_fa_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr<float>(), B, Sq, Skv, H,
                              (float)scale, (int)variant, cb200_error_word(q.get_device()), at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(rc == 0, "fa_fwd launch failed with code ", rc);
  return {o, lse};
}
std::tuple<Tensor, Tensor> fa_fwd(const Tensor& q, const Tensor& k, const Tensor& v, double scale) {
  return fa_fwd_variant(q, k, v, scale, 0);
}

// gradients of softmax(q k^T scale) v given the forward's output and log-sum-exp
std::tuple<Tensor, Tensor, Tensor> fa_bwd(const Tensor& d_o, const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& o,
                                          const Tensor& lse, double scale) {
  check_qkv(d_o, "do");
  check_qkv(q, "q");
  check_qkv(k, "k");
  check_qkv(v, "v");
  check_qkv(o, "o");
  TORCH_CHECK(lse.is_cuda() && lse.scalar_type() == at::kFloat && lse.is_contiguous(), "lse must be contiguous fp32 [B,H,Sq]");
  c10::cuda::CUDAGuard g(q.device());
  const int B = (int)q.size(0), Sq = (int)q.size(1), H = (int)q.size(2), Skv = (int)k.size(1);
  Tensor dq = at::empty_like(q), dk = at::empty_like(k), dv = at::empty_like(v);
  Tensor scratch = at::empty({(int64_t)cb200_fa_bwd_scratch_floats(B, Sq, H)}, q.options().dtype(at::kFloat));
  const int rc = cb200_fa_bwd(d_o.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr<float>(),
                              dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), scratch.data_ptr<float>(), B, Sq, Skv, H, (float)scale,
                              cb200_error_word(q.get_device()), at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(rc == 0, "fa_bwd launch failed with code ", rc);
  return {dq, dk, dv};
}
}  // namespace

void register_attention_ops(torch::Library& m) {
  m.def("fa_fwd(Tensor q, Tensor k, Tensor v, float scale) -> (Tensor, Tensor)", &fa_fwd);
  m.def("fa_bwd(Tensor do, Tensor q, Tensor k, Tensor v, Tensor o, Tensor lse, float scale) -> (Tensor, Tensor, Tensor)", &fa_bwd);
  m.def("fa_fwd_variant(Tensor q, Tensor k, Tensor v, float scale, int variant) -> (Tensor, Tensor)", &fa_fwd_variant);
}
