// Attention operators of torch.ops.cosmos_b200.

#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include <tuple>
#include <vector>

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
                              (float)scale, (int)variant, cb200_error_word(q.get_device()),
                              at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(rc == 0, "fa_fwd launch failed with code ", rc);
  return {o, lse};
}
// Attention on local heads of the whole sequence with the head->sequence exchange as its epilogue: output row s goes to
// out_ptrs[s / (Sq/P)], a buffer [B, Sq/P, P*H, 128] on that rank, at heads [rank*H, rank*H + H).  Returns lse.
Tensor fa_fwd_scatter_seq_peer(const Tensor& q, const Tensor& k, const Tensor& v, double scale, c10::ArrayRef<int64_t> out_ptrs,
                               int64_t rank) {
  check_qkv(q, "q");
  check_qkv(k, "k");
  check_qkv(v, "v");
  TORCH_CHECK(k.sizes() == v.sizes() && q.size(0) == k.size(0) && q.size(2) == k.size(2), "q/k/v shape mismatch");
  const int P = (int)out_ptrs.size();
  TORCH_CHECK(P >= 1 && P <= 8 && q.size(1) % P == 0, "sequence must divide over 1..8 peers");
  c10::cuda::CUDAGuard g(q.device());
  const int B = (int)q.size(0), Sq = (int)q.size(1), H = (int)q.size(2), Skv = (int)k.size(1);
  Tensor lse = at::empty({B, H, Sq}, q.options().dtype(at::kFloat));
  std::vector<int64_t> p(out_ptrs.begin(), out_ptrs.end());
  const int rc = cb200_fa_fwd_scatter_seq(q.data_ptr(), k.data_ptr(), v.data_ptr(), p.data(), P, (int)rank, lse.data_ptr<float>(), B,
                                          Sq, Skv, H, (float)scale, cb200_error_word(q.get_device()),
                                          at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(rc == 0, "fa_fwd (sequence-scatter epilogue) launch failed with code ", rc);
  return lse;
}

// Neighbourhood attention on a T x H x W token grid in natural (t, h, w) order; the kernel tiles it 4 x 4 x 8 by itself.
// kv_idx [n_blocks, max_n] int32, kv_cnt [n_blocks] int32 (n_blocks = ceil(n_tiles / 2)); bt/bh/bw: uint8 visibility tables
// [T, nT], [H, nH], [W, nW].  Returns (o, lse).
std::tuple<Tensor, Tensor> fa_fwd_na(const Tensor& q, const Tensor& k, const Tensor& v, double scale, const Tensor& kv_idx,
                                     const Tensor& kv_cnt, const Tensor& bt, const Tensor& bh, const Tensor& bw) {
  check_qkv(q, "q");
  check_qkv(k, "k");
  check_qkv(v, "v");
  TORCH_CHECK(q.sizes() == k.sizes() && k.sizes() == v.sizes(), "neighbourhood attention is self-attention: equal shapes");
  const int B = (int)q.size(0), S = (int)q.size(1), H = (int)q.size(2);
  TORCH_CHECK(S % 128 == 0, "sequence must be whole 128-token tiles");
  const int n_tiles = S / 128, n_blocks = (n_tiles + 1) / 2;
  for (const Tensor* t : {&kv_idx, &kv_cnt})
    TORCH_CHECK(t->is_cuda() && t->scalar_type() == at::kInt && t->is_contiguous(), "tile lists must be contiguous CUDA int32");
  for (const Tensor* t : {&bt, &bh, &bw})
    TORCH_CHECK(t->is_cuda() && t->scalar_type() == at::kByte && t->is_contiguous() && t->dim() == 2, "visibility tables: CUDA uint8 2-D");
  TORCH_CHECK(kv_idx.dim() == 2 && kv_idx.size(0) == n_blocks && kv_cnt.numel() == n_blocks, "one tile list per query block");
  const int nT = (int)bt.size(1), nH = (int)bh.size(1), nW = (int)bw.size(1);
  TORCH_CHECK((int64_t)nT * nH * nW == n_tiles && bt.size(0) == 4 * nT && bh.size(0) == 4 * nH && bw.size(0) == 8 * nW,
              "tables do not match the tile grid");
  c10::cuda::CUDAGuard g(q.device());
  Tensor o = at::empty_like(q);
  Tensor lse = at::empty({B, H, S}, q.options().dtype(at::kFloat));
  const int rc = cb200_fa_fwd_na(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr<float>(), B, S, H, (float)scale,
                                 kv_idx.data_ptr<int>(), kv_cnt.data_ptr<int>(), (int)kv_idx.size(1), bt.data_ptr<uint8_t>(),
                                 bh.data_ptr<uint8_t>(), bw.data_ptr<uint8_t>(), nT, nH, nW, cb200_error_word(q.get_device()),
                                 at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(rc == 0, "fa_fwd_na launch failed with code ", rc);
  return {o, lse};
}

// Gradients of the neighbourhood attention. Every tensor is in TILE order (tile = one 4 x 4 x 8 token box, row dt*32 + dh*8 + dw;
// ``TilePlan.to_tiles``), lse [B, H, S] in the same order. q_list [S/128, max_n] int32: the query tiles that see each key tile
// (top bit set: the whole pair is visible), q_cnt [S/128]; bt/bh/bw: uint8 [4 nT, nT], [4 nH, nH], [8 nW, nW] with, for one key
// coordinate and one query tile, the visibility bits of the tile's query coordinates. Returns (dq, dk, dv) in tile order.
std::tuple<Tensor, Tensor, Tensor> fa_bwd_na(const Tensor& d_o, const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& o,
                                             const Tensor& lse, double scale, const Tensor& q_list, const Tensor& q_cnt,
                                             const Tensor& bt, const Tensor& bh, const Tensor& bw) {
  check_qkv(d_o, "do");
  check_qkv(q, "q");
  check_qkv(k, "k");
  check_qkv(v, "v");
  check_qkv(o, "o");
  TORCH_CHECK(q.sizes() == k.sizes() && k.sizes() == v.sizes() && o.sizes() == q.sizes() && d_o.sizes() == q.sizes(),
              "neighbourhood attention is self-attention: equal shapes");
  const int B = (int)q.size(0), S = (int)q.size(1), H = (int)q.size(2);
  TORCH_CHECK(S % 128 == 0, "sequence must be whole 128-token tiles");
  const int n_tiles = S / 128;
  TORCH_CHECK(lse.is_cuda() && lse.scalar_type() == at::kFloat && lse.is_contiguous() && lse.numel() == (int64_t)B * H * S,
              "lse must be contiguous fp32 [B,H,S]");
  for (const Tensor* t : {&q_list, &q_cnt})
    TORCH_CHECK(t->is_cuda() && t->scalar_type() == at::kInt && t->is_contiguous(), "tile lists must be contiguous CUDA int32");
  for (const Tensor* t : {&bt, &bh, &bw})
    TORCH_CHECK(t->is_cuda() && t->scalar_type() == at::kByte && t->is_contiguous() && t->dim() == 2, "visibility tables: CUDA uint8 2-D");
  TORCH_CHECK(q_list.dim() == 2 && q_list.size(0) == n_tiles && q_list.size(1) >= 1 && q_cnt.numel() == n_tiles,
              "one query-tile list per key tile");
  const int nT = (int)bt.size(1), nH = (int)bh.size(1), nW = (int)bw.size(1);
  TORCH_CHECK((int64_t)nT * nH * nW == n_tiles && bt.size(0) == 4 * nT && bh.size(0) == 4 * nH && bw.size(0) == 8 * nW,
              "tables do not match the tile grid");
  c10::cuda::CUDAGuard g(q.device());
  Tensor dq = at::empty_like(q), dk = at::empty_like(k), dv = at::empty_like(v);
  Tensor scratch = at::empty({(int64_t)cb200_fa_bwd_na_scratch_floats(B, S, H)}, q.options().dtype(at::kFloat));
  const int rc = cb200_fa_bwd_na(d_o.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr<float>(),
                                 dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), scratch.data_ptr<float>(), B, S, H, (float)scale,
                                 q_list.data_ptr<int>(), q_cnt.data_ptr<int>(), (int)q_list.size(1), bt.data_ptr<uint8_t>(),
                                 bh.data_ptr<uint8_t>(), bw.data_ptr<uint8_t>(), nT, nH, nW, cb200_error_word(q.get_device()),
                                 at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(rc == 0, "fa_bwd_na launch failed with code ", rc);
  return {dq, dk, dv};
}

std::tuple<Tensor, Tensor> fa_fwd(const Tensor& q, const Tensor& k, const Tensor& v, double scale) {
  return fa_fwd_variant(q, k, v, scale, 0);
}

// gradients of softmax(q k^T scale) v given the forward's output and log-sum-exp
// variant 0: by problem size; 1: two deterministic kernels; 2: single pass, 128 x 64 sub-tiles; 3: single pass, 128 x 128 tiles
// (2 and 3 accumulate dQ in fp32 with reductions in global memory: run-to-run differences of the last bit are possible)
std::tuple<Tensor, Tensor, Tensor> fa_bwd_variant(const Tensor& d_o, const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& o,
                                                  const Tensor& lse, double scale, int64_t variant) {
  check_qkv(d_o, "do");
  check_qkv(q, "q");
  check_qkv(k, "k");
  check_qkv(v, "v");
  check_qkv(o, "o");
  TORCH_CHECK(lse.is_cuda() && lse.scalar_type() == at::kFloat && lse.is_contiguous(), "lse must be contiguous fp32 [B,H,Sq]");
  c10::cuda::CUDAGuard g(q.device());
  const int B = (int)q.size(0), Sq = (int)q.size(1), H = (int)q.size(2), Skv = (int)k.size(1);
  Tensor dq = at::empty_like(q), dk = at::empty_like(k), dv = at::empty_like(v);
  Tensor scratch = at::empty({(int64_t)cb200_fa_bwd_scratch_floats_v(B, Sq, Skv, H, (int)variant)}, q.options().dtype(at::kFloat));
  const int rc = cb200_fa_bwd_v(d_o.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr<float>(),
                                dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), scratch.data_ptr<float>(), B, Sq, Skv, H, (float)scale,
                                (int)variant, cb200_error_word(q.get_device()), at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(rc == 0, "fa_bwd launch failed with code ", rc);
  return {dq, dk, dv};
}

std::tuple<Tensor, Tensor, Tensor> fa_bwd(const Tensor& d_o, const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& o,
                                          const Tensor& lse, double scale) {
  return fa_bwd_variant(d_o, q, k, v, o, lse, scale, 0);
}
// tangent of the attention output given the primal output and log-sum-exp of the forward kernel
Tensor fa_jvp_tangent(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& tq, const Tensor& tk, const Tensor& tv,
                      const Tensor& o, const Tensor& lse, double scale) {
  check_qkv(q, "q");
  check_qkv(k, "k");
  check_qkv(v, "v");
  check_qkv(tq, "tq");
  check_qkv(tk, "tk");
  check_qkv(tv, "tv");
  check_qkv(o, "o");
  TORCH_CHECK(tq.sizes() == q.sizes() && tk.sizes() == k.sizes() && tv.sizes() == v.sizes(), "tangent shapes must match the primals");
  TORCH_CHECK(lse.is_cuda() && lse.scalar_type() == at::kFloat && lse.is_contiguous(), "lse must be contiguous fp32 [B,H,Sq]");
  c10::cuda::CUDAGuard g(q.device());
  Tensor to = at::empty_like(q);
  const int B = (int)q.size(0), Sq = (int)q.size(1), H = (int)q.size(2), Skv = (int)k.size(1);
  const int rc = cb200_fa_jvp(q.data_ptr(), k.data_ptr(), v.data_ptr(), tq.data_ptr(), tk.data_ptr(), tv.data_ptr(), o.data_ptr(),
                              lse.data_ptr<float>(), to.data_ptr(), B, Sq, Skv, H, (float)scale, cb200_error_word(q.get_device()),
                              at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(rc == 0, "fa_jvp launch failed with code ", rc);
  return to;
}

// primal output, tangent output and log-sum-exp of attention for tangents (tq, tk, tv): forward kernel, then one JVP pass
std::tuple<Tensor, Tensor, Tensor> fa_jvp(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& tq, const Tensor& tk,
                                          const Tensor& tv, double scale) {
  auto ol = fa_fwd(q, k, v, scale);
  const Tensor& o = std::get<0>(ol);
  const Tensor& lse = std::get<1>(ol);
  return {o, fa_jvp_tangent(q, k, v, tq, tk, tv, o, lse, scale), lse};
}

}  // namespace

void register_attention_ops(torch::Library& m) {
  // Schemas only: the kernels are registered under the CUDA dispatch key below so that dispatch modes (selective
  // activation checkpointing keeps the attention output by intercepting this op) see the call.
  m.def("fa_fwd(Tensor q, Tensor k, Tensor v, float scale) -> (Tensor, Tensor)");
  m.def("fa_fwd_na(Tensor q, Tensor k, Tensor v, float scale, Tensor kv_idx, Tensor kv_cnt, Tensor bt, Tensor bh, Tensor bw) -> "
        "(Tensor, Tensor)");
  m.def("fa_bwd_na(Tensor do, Tensor q, Tensor k, Tensor v, Tensor o, Tensor lse, float scale, Tensor q_list, Tensor q_cnt, Tensor bt, "
        "Tensor bh, Tensor bw) -> (Tensor, Tensor, Tensor)", &fa_bwd_na);
  m.def("fa_fwd_scatter_seq_peer(Tensor q, Tensor k, Tensor v, float scale, int[] out_ptrs, int rank) -> Tensor",
        &fa_fwd_scatter_seq_peer);
  m.def("fa_bwd(Tensor do, Tensor q, Tensor k, Tensor v, Tensor o, Tensor lse, float scale) -> (Tensor, Tensor, Tensor)");
  m.def("fa_fwd_variant(Tensor q, Tensor k, Tensor v, float scale, int variant) -> (Tensor, Tensor)");
  m.def("fa_jvp(Tensor q, Tensor k, Tensor v, Tensor tq, Tensor tk, Tensor tv, float scale) -> (Tensor, Tensor, Tensor)");
  m.def("fa_jvp_tangent(Tensor q, Tensor k, Tensor v, Tensor tq, Tensor tk, Tensor tv, Tensor o, Tensor lse, float scale) -> Tensor");
  m.def("fa_bwd_variant(Tensor do, Tensor q, Tensor k, Tensor v, Tensor o, Tensor lse, float scale, int variant) -> (Tensor, Tensor, Tensor)");
}

TORCH_LIBRARY_IMPL(cosmos_b200, CUDA, m) {
  m.impl("fa_fwd", &fa_fwd);
  m.impl("fa_fwd_na", &fa_fwd_na);
  m.impl("fa_bwd", &fa_bwd);
  m.impl("fa_fwd_variant", &fa_fwd_variant);
  m.impl("fa_bwd_variant", &fa_bwd_variant);
  m.impl("fa_jvp", &fa_jvp);
  m.impl("fa_jvp_tangent", &fa_jvp_tangent);
}
