// Peer-memory (NVLink) operators of torch.ops.cosmos_b200; the kernels are in peer.cu.
// Peer pointers arrive as Python int lists (virtual addresses of the same symmetric buffer on each rank).

#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include <vector>

#include "launchers.h"

int* cb200_error_word(int device);

namespace {
using at::Tensor;

inline cudaStream_t stream() { return at::cuda::getCurrentCUDAStream().stream(); }

// every operand that a kernel indexes through a raw pointer is checked here: a wrong dtype, device, layout or size must be a
// Python error, not an out-of-bounds access to this GPU's or a peer's memory
void check_shard(const Tensor& t, const char* name, const Tensor& like) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kFloat && t.is_contiguous(), name, " must be a contiguous fp32 CUDA tensor");
  TORCH_CHECK(t.device() == like.device() && t.numel() == like.numel(), name, " must match the master shard in device and size");
}

void check_segs(const Tensor& segs, const Tensor& like) {
  TORCH_CHECK(segs.is_cuda() && segs.scalar_type() == at::kLong && segs.is_contiguous() && segs.dim() == 2 && segs.size(1) == 4 &&
                  segs.size(0) >= 1,
              "segment table must be a contiguous int64 CUDA tensor [n, 4]");
  TORCH_CHECK(segs.device() == like.device(), "segment table is on another device than the shard");
}

void check_rope(const c10::optional<Tensor>& cosv, const c10::optional<Tensor>& sinv, int64_t S, int64_t HD, const Tensor& x) {
  TORCH_CHECK(cosv.has_value() == sinv.has_value(), "cos and sin come together");
  if (!cosv.has_value()) return;
  for (const Tensor* t : {&*cosv, &*sinv}) {
    TORCH_CHECK(t->is_cuda() && t->scalar_type() == at::kFloat && t->is_contiguous() && t->device() == x.device(),
                "cos/sin must be contiguous fp32 CUDA tensors on the device of x");
    TORCH_CHECK(t->dim() == 2 && t->size(0) == S && t->size(1) == HD / 2, "cos/sin must be [S, D/2] for the local sequence slice");
  }
}

std::vector<int64_t> ptr_vec(c10::ArrayRef<int64_t> v) {
  TORCH_CHECK(v.size() >= 1 && v.size() <= 8, "1..8 peers supported");
  return std::vector<int64_t>(v.begin(), v.end());
}

void peer_barrier(c10::ArrayRef<int64_t> flag_ptrs, int64_t rank, int64_t epoch, int64_t device, int64_t max_spins) {
  c10::cuda::CUDAGuard g((c10::DeviceIndex)device);
  auto p = ptr_vec(flag_ptrs);
  cb200_peer_barrier(p.data(), (int)rank, (int)p.size(), (unsigned)epoch, (unsigned)max_spins, cb200_error_word((int)device), stream());
}

// segs: int64 CUDA tensor [nseg, 4] = (full_offset, stride, shard_offset, numel)
void rs_cast_norm_peer(c10::ArrayRef<int64_t> grad_ptrs, const Tensor& segs, Tensor g32, Tensor unit_sumsq,
                       const c10::optional<Tensor>& total_sumsq, int64_t rank, double scale) {
  TORCH_CHECK(g32.is_cuda() && g32.scalar_type() == at::kFloat && g32.is_contiguous(), "g32 must be a contiguous fp32 CUDA tensor");
  check_segs(segs, g32);
  check_shard(unit_sumsq, "unit_sumsq", unit_sumsq);
  TORCH_CHECK(unit_sumsq.numel() >= 1 && unit_sumsq.device() == g32.device(), "unit_sumsq: one float on the device of g32");
  if (total_sumsq.has_value())
    TORCH_CHECK(total_sumsq->is_cuda() && total_sumsq->scalar_type() == at::kFloat && total_sumsq->numel() >= 1 &&
                    total_sumsq->device() == g32.device(), "total_sumsq: one float on the device of g32");
  c10::cuda::CUDAGuard g(g32.device());
  auto p = ptr_vec(grad_ptrs);
  TORCH_CHECK(rank >= 0 && rank < (int64_t)p.size(), "rank out of range");
  const int nseg = (int)segs.size(0);
  Tensor partials = at::empty({(int64_t)cb200_rs_blocks_x() * nseg}, g32.options());
  cb200_rs_cast_norm_peer(p.data(), segs.data_ptr(), nseg, g32.data_ptr<float>(), partials.data_ptr<float>(),
                          unit_sumsq.data_ptr<float>(), total_sumsq.has_value() ? total_sumsq->data_ptr<float>() : nullptr,
                          (int)rank, (int)p.size(), (float)scale, stream());
}

void adamw_push_peer(c10::ArrayRef<int64_t> full_ptrs, c10::ArrayRef<int64_t> sumsq_ptrs, const Tensor& segs, Tensor master,
                     const Tensor& grad, Tensor m, Tensor v, const c10::optional<Tensor>& ema, int64_t rank, double max_norm,
                     double lr, double beta1, double beta2, double eps, double wd, int64_t step, double ema_beta,
                     const c10::optional<Tensor>& norm_out) {
  check_shard(master, "master", master);
  check_shard(grad, "grad", master);
  check_shard(m, "exp_avg", master);
  check_shard(v, "exp_avg_sq", master);
  if (ema.has_value()) check_shard(*ema, "ema", master);
  check_segs(segs, master);
  if (norm_out.has_value())
    TORCH_CHECK(norm_out->is_cuda() && norm_out->scalar_type() == at::kFloat && norm_out->numel() >= 1 &&
                    norm_out->device() == master.device(), "norm_out: one float on the device of the shard");
  c10::cuda::CUDAGuard g(master.device());
  auto fp = ptr_vec(full_ptrs);
  auto sp = ptr_vec(sumsq_ptrs);
  TORCH_CHECK(fp.size() == sp.size(), "pointer lists differ in length");
  TORCH_CHECK(rank >= 0 && rank < (int64_t)fp.size(), "rank out of range");
  cb200_adamw_push_peer(fp.data(), sp.data(), segs.data_ptr(), (int)segs.size(0), master.data_ptr<float>(), grad.data_ptr<float>(),
                        m.data_ptr<float>(), v.data_ptr<float>(), ema.has_value() ? ema->data_ptr<float>() : nullptr, (int)rank,
                        (int)fp.size(), (float)max_norm, (float)lr, (float)beta1, (float)beta2, (float)eps, (float)wd, step,
                        (float)ema_beta, norm_out.has_value() ? norm_out->data_ptr<float>() : nullptr, stream());
}

// x [B,S,H,HD] -> peers' buffers laid out [B, P*S, H/P, HD]; returns rstd [B,S,H] when norm is applied
Tensor a2a_scatter_heads_peer(const Tensor& x, c10::ArrayRef<int64_t> out_ptrs, const c10::optional<Tensor>& w,
                              const c10::optional<Tensor>& cosv, const c10::optional<Tensor>& sinv, int64_t rank, double eps) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.is_contiguous() && x.dim() == 4, "x must be bf16 [B,S,H,HD]");
  c10::cuda::CUDAGuard g(x.device());
  auto p = ptr_vec(out_ptrs);
  const int64_t B = x.size(0), S = x.size(1), H = x.size(2), HD = x.size(3);
  TORCH_CHECK((HD == 128 || HD == 64) && H % (int64_t)p.size() == 0, "head_dim 64/128 and heads divisible by peers");
  TORCH_CHECK(rank >= 0 && rank < (int64_t)p.size(), "rank out of range");
  if (w.has_value()) {
    TORCH_CHECK(w->is_cuda() && w->device() == x.device() && w->numel() == HD, "norm weight must hold head_dim values on the device of x");
    check_rope(cosv, sinv, S, HD, x);
  } else {
    TORCH_CHECK(!cosv.has_value() && !sinv.has_value(), "RoPE is applied only together with the norm");
  }
  Tensor rstd = at::empty({w.has_value() ? B * S * H : 0}, x.options().dtype(at::kFloat));
  Tensor wf;
  const float* wp = nullptr;
  if (w.has_value()) {
    wf = w->to(at::kFloat).contiguous();
    wp = wf.data_ptr<float>();
  }
  cb200_a2a_scatter_heads_peer(x.data_ptr(), p.data(), wp, cosv.has_value() ? cosv->data_ptr<float>() : nullptr,
                               sinv.has_value() ? sinv->data_ptr<float>() : nullptr,
                               w.has_value() ? rstd.data_ptr<float>() : nullptr, B * S * H, (int)S, (int)H, (int)HD, (int)rank,
                               (int)p.size(), w.has_value() ? 1 : 0, (float)eps, stream());
  return rstd;
}

Tensor a2a_gather_seq_peer(c10::ArrayRef<int64_t> src_ptrs, int64_t B, int64_t S, int64_t H, int64_t HD, int64_t rank,
                           const Tensor& like) {
  TORCH_CHECK(like.is_cuda(), "like must be a CUDA tensor");
  c10::cuda::CUDAGuard g(like.device());
  auto p = ptr_vec(src_ptrs);
  TORCH_CHECK(rank >= 0 && rank < (int64_t)p.size() && B >= 1 && S >= 1 && H >= 1 && (HD == 64 || HD == 128) &&
                  H % (int64_t)p.size() == 0, "bad exchange shape");
  Tensor out = at::empty({B, S, H, HD}, like.options().dtype(at::kBFloat16));
  cb200_a2a_gather_seq_peer(p.data(), out.data_ptr(), B, (int)S, (int)H, (int)HD, (int)rank, (int)p.size(), stream());
  return out;
}

int sm_count_peer(int device) {
  static int cache[64] = {0};
  if (cache[device] == 0) cache[device] = at::cuda::getDeviceProperties(device)->multiProcessorCount;
  return cache[device];
}

// Small parameters of a unit, all-gathered by peer reads: segs [n, 4] as for the other segment kernels; `full` is the local
// full-layout buffer that receives every rank's chunk.
void gather_slots_peer(c10::ArrayRef<int64_t> shard_ptrs, const Tensor& segs, Tensor full) {
  TORCH_CHECK(full.is_cuda() && full.scalar_type() == at::kBFloat16 && full.is_contiguous(), "full must be a contiguous CUDA bf16 tensor");
  check_segs(segs, full);
  c10::cuda::CUDAGuard g(full.device());
  auto p = ptr_vec(shard_ptrs);
  cb200_gather_slots_peer(p.data(), segs.data_ptr(), (int)segs.size(0), full.data_ptr(), (int)p.size(), stream());
}

// FSDP all-gather fused into the consuming GEMM. `ws` [rows, ld] is the local full-size home of a weight whose rows are sharded
// over the ranks (shard_ptrs[r]: rank r's rows [r * chunk_rows, ...), row-major); the kernel fills it while it computes.
//   trans_b = false: returns x [M, ld] @ W^T  (+ bias, optional GELU; `pre` receives the pre-activation when given)
//   trans_b = true : returns x [M, rows] @ W  (dgrad)
Tensor gemm_bf16_gather(const Tensor& x, Tensor ws, c10::ArrayRef<int64_t> shard_ptrs, int64_t chunk_rows, Tensor counters,
                        const c10::optional<Tensor>& bias, int64_t act, bool trans_b, const c10::optional<Tensor>& pre) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.is_contiguous() && x.dim() == 2, "x must be contiguous CUDA bf16 [M, K]");
  TORCH_CHECK(ws.is_cuda() && ws.scalar_type() == at::kBFloat16 && ws.is_contiguous() && ws.dim() == 2 && ws.device() == x.device(),
              "ws must be contiguous CUDA bf16 [rows, ld] on the device of x");
  const int64_t rows = ws.size(0), ld = ws.size(1), M = x.size(0);
  TORCH_CHECK(x.size(1) == (trans_b ? rows : ld), "contraction dims differ");
  TORCH_CHECK(ld % 8 == 0 && x.size(1) % 8 == 0, "row strides must be multiples of 16 bytes");
  auto p = ptr_vec(shard_ptrs);
  TORCH_CHECK(chunk_rows >= 1 && chunk_rows * (int64_t)p.size() >= rows, "shards do not cover the weight");
  const int64_t n_groups = (rows + 255) / 256;
  TORCH_CHECK(counters.is_cuda() && counters.scalar_type() == at::kInt && counters.is_contiguous() && counters.numel() >= n_groups &&
                  counters.device() == x.device(), "counters: CUDA int32, one per 256 rows");
  c10::cuda::CUDAGuard g(x.device());
  Tensor c = at::empty({M, trans_b ? ld : rows}, x.options());
  Tensor bias_c;
  const void* bias_p = nullptr;
  if (bias.has_value()) {
    TORCH_CHECK(!trans_b, "bias belongs to the forward form");
    bias_c = bias->to(at::kBFloat16).contiguous();
    TORCH_CHECK(bias_c.numel() == rows && bias_c.device() == x.device(), "bias must be [rows]");
    bias_p = bias_c.data_ptr();
  }
  void* pre_p = nullptr;
  if (pre.has_value()) {
    TORCH_CHECK(pre->is_cuda() && pre->scalar_type() == at::kBFloat16 && pre->is_contiguous() && pre->numel() == c.numel() && act == 1,
                "pre: bf16 tensor of the output's size, only with the GELU epilogue");
    pre_p = pre->data_ptr();
  }
  const int dev = x.get_device();
  const int rc = cb200_gemm_bf16_gather(x.data_ptr(), ws.data_ptr(), c.data_ptr(), (int)M, (int)rows, (int)ld, trans_b ? 1 : 0, p.data(),
                                        (int)p.size(), (int)chunk_rows, counters.data_ptr<int>(), bias_p, (int)act, pre_p,
                                        cb200_error_word(dev), sm_count_peer(dev), stream());
  TORCH_CHECK(rc == 0, "gather GEMM launch failed with code ", rc);
  return c;
}

}  // namespace

void register_peer_ops(torch::Library& m) {
  m.def("gather_slots_peer(int[] shard_ptrs, Tensor segs, Tensor(a!) full) -> ()", &gather_slots_peer);
  m.def("gemm_bf16_gather(Tensor x, Tensor(a!) ws, int[] shard_ptrs, int chunk_rows, Tensor(b!) counters, Tensor? bias, int act, "
        "bool trans_b, Tensor(c!)? pre) -> Tensor", &gemm_bf16_gather);
  m.def("peer_barrier(int[] flag_ptrs, int rank, int epoch, int device, int max_spins) -> ()", &peer_barrier);
  m.def("rs_cast_norm_peer(int[] grad_ptrs, Tensor segs, Tensor(a!) g32, Tensor(b!) unit_sumsq, Tensor(c!)? total_sumsq, int rank, "
        "float scale) -> ()", &rs_cast_norm_peer);
  m.def("adamw_push_peer(int[] full_ptrs, int[] sumsq_ptrs, Tensor segs, Tensor(a!) master, Tensor grad, Tensor(b!) m, Tensor(c!) v, "
        "Tensor(d!)? ema, int rank, float max_norm, float lr, float beta1, float beta2, float eps, float wd, int step, "
        "float ema_beta, Tensor(e!)? norm_out) -> ()", &adamw_push_peer);
  m.def("a2a_scatter_heads_peer(Tensor x, int[] out_ptrs, Tensor? w, Tensor? cos, Tensor? sin, int rank, float eps) -> Tensor",
        &a2a_scatter_heads_peer);
  m.def("a2a_gather_seq_peer(int[] src_ptrs, int B, int S, int H, int HD, int rank, Tensor like) -> Tensor", &a2a_gather_seq_peer);
}
