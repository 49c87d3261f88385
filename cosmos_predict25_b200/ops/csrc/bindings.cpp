// torch.ops.cosmos_b200.* : registration of the sm_100a kernels with the PyTorch dispatcher.
// Only this file sees torch headers; kernels are reached through the C launchers in launchers.h.

#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include <tuple>

#include "launchers.h"

namespace {

using at::Tensor;

inline cudaStream_t stream() { return at::cuda::getCurrentCUDAStream().stream(); }

inline void check_bf16(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
  TORCH_CHECK(t.scalar_type() == at::kBFloat16, name, " must be bfloat16");
  TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
}
inline void check_f32(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
  TORCH_CHECK(t.scalar_type() == at::kFloat, name, " must be float32");
  TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
}

constexpr int kRowsPerCta = 32;
constexpr int kRowsPerWarp = CB200_RMSNORM_BWD_ROWS_PER_WARP;

}  // namespace

// per-device error word written by kernels whose bounded waits gave up
int* cb200_error_word(int device) {
  static int* words[64] = {nullptr};
  if (words[device] == nullptr) {
    C10_CUDA_CHECK(cudaMalloc(&words[device], sizeof(int)));
    C10_CUDA_CHECK(cudaMemset(words[device], 0, sizeof(int)));
  }
  return words[device];
}

namespace {
inline int* error_word(int device) { return cb200_error_word(device); }

std::tuple<Tensor, Tensor, Tensor> ln_modulate_fwd(const Tensor& x, const Tensor& shift, const Tensor& scale, int64_t L,
                                                   double eps) {
  check_bf16(x, "x");
  check_f32(shift, "shift");
  check_f32(scale, "scale");
  c10::cuda::CUDAGuard g(x.device());
  const int64_t rows = x.size(0), D = x.size(1);
  TORCH_CHECK(D % 8 == 0 && D <= 8192, "channel dim must be a multiple of 8 and <= 8192");
  TORCH_CHECK(rows % L == 0 && shift.size(0) == rows / L && shift.size(1) == D, "shift/scale must be [rows/L, D]");
  Tensor y = at::empty_like(x);
  Tensor mean = at::empty({rows}, x.options().dtype(at::kFloat));
  Tensor rstd = at::empty({rows}, x.options().dtype(at::kFloat));
  cb200_ln_modulate_fwd(x.data_ptr(), shift.data_ptr<float>(), scale.data_ptr<float>(), y.data_ptr(), mean.data_ptr<float>(),
                        rstd.data_ptr<float>(), rows, (int)D, (int)L, (float)eps, stream());
  return {y, mean, rstd};
}

std::tuple<Tensor, Tensor, Tensor> ln_modulate_bwd(const Tensor& dy, const Tensor& x, const Tensor& mean, const Tensor& rstd,
                                                   const Tensor& scale, int64_t L) {
  check_bf16(dy, "dy");
  check_bf16(x, "x");
  check_f32(scale, "scale");
  c10::cuda::CUDAGuard g(x.device());
  const int64_t rows = x.size(0), D = x.size(1), frames = rows / L;
  Tensor dx = at::empty_like(x);
  Tensor dshift = at::empty({frames, D}, scale.options());
  Tensor dscale = at::empty({frames, D}, scale.options());
  const int G = cb200_ln_groups_per_frame((int)L, kRowsPerCta);
  Tensor partials = at::empty({frames * G, 2, D}, scale.options());
  cb200_ln_modulate_bwd(dy.data_ptr(), x.data_ptr(), mean.data_ptr<float>(), rstd.data_ptr<float>(), scale.data_ptr<float>(),
                        dx.data_ptr(), dshift.data_ptr<float>(), dscale.data_ptr<float>(), partials.data_ptr<float>(), frames,
                        (int)D, (int)L, kRowsPerCta, stream());
  return {dx, dshift, dscale};
}

Tensor gate_residual_fwd(const Tensor& x, const Tensor& gate, const Tensor& y, int64_t L) {
  check_bf16(x, "x");
  check_bf16(y, "y");
  check_f32(gate, "gate");
  c10::cuda::CUDAGuard g(x.device());
  const int64_t rows = x.size(0), D = x.size(1);
  TORCH_CHECK(D % 8 == 0 && gate.size(0) == rows / L && gate.size(1) == D, "gate must be [rows/L, D]");
  Tensor out = at::empty_like(x);
  cb200_gate_residual_fwd(x.data_ptr(), gate.data_ptr<float>(), y.data_ptr(), out.data_ptr(), rows, (int)D, (int)L, stream());
  return out;
}

std::tuple<Tensor, Tensor> gate_residual_bwd(const Tensor& dout, const Tensor& gate, const Tensor& y, int64_t L) {
  check_bf16(dout, "dout");
  check_bf16(y, "y");
  check_f32(gate, "gate");
  c10::cuda::CUDAGuard g(y.device());
  const int64_t rows = y.size(0), D = y.size(1), frames = rows / L;
  TORCH_CHECK(D <= 8192, "channel dim must be <= 8192");
  Tensor dy = at::empty_like(y);
  Tensor dgate = at::empty({frames, D}, gate.options());
  const int G = cb200_ln_groups_per_frame((int)L, kRowsPerCta);
  Tensor partials = at::empty({frames * G, D}, gate.options());
  cb200_gate_residual_bwd(dout.data_ptr(), gate.data_ptr<float>(), y.data_ptr(), dy.data_ptr(), dgate.data_ptr<float>(),
                          partials.data_ptr<float>(), frames, (int)D, (int)L, kRowsPerCta, stream());
  return {dy, dgate};
}

std::tuple<Tensor, Tensor> rmsnorm_rope_fwd(const Tensor& x, const Tensor& w, const c10::optional<Tensor>& cosv,
                                            const c10::optional<Tensor>& sinv, double eps) {
  check_bf16(x, "x");
  TORCH_CHECK(x.dim() == 4, "x must be [B, S, H, D]");
  c10::cuda::CUDAGuard g(x.device());
  const int64_t B = x.size(0), S = x.size(1), H = x.size(2), HD = x.size(3);
  TORCH_CHECK(HD == 128 || HD == 64, "head_dim must be 64 or 128");
  Tensor wf = w.to(at::kFloat).contiguous();
  const float* cp = nullptr;
  const float* sp = nullptr;
  if (cosv.has_value()) {
    check_f32(*cosv, "cos");
    check_f32(*sinv, "sin");
    TORCH_CHECK(cosv->size(0) == S && cosv->size(1) == HD / 2, "cos/sin must be [S, D/2]");
    cp = cosv->data_ptr<float>();
    sp = sinv->data_ptr<float>();
  }
  Tensor y = at::empty_like(x);
  Tensor rstd = at::empty({B, S, H}, x.options().dtype(at::kFloat));
  cb200_rmsnorm_rope_fwd(x.data_ptr(), wf.data_ptr<float>(), cp, sp, y.data_ptr(), rstd.data_ptr<float>(), B * S * H, (int)S,
                         (int)H, (int)HD, (float)eps, stream());
  return {y, rstd};
}

std::tuple<Tensor, Tensor> rmsnorm_rope_bwd(const Tensor& dy, const Tensor& x, const Tensor& w, const Tensor& rstd,
                                            const c10::optional<Tensor>& cosv, const c10::optional<Tensor>& sinv) {
  check_bf16(dy, "dy");
  check_bf16(x, "x");
  TORCH_CHECK(x.dim() == 4 && dy.sizes() == x.sizes() && dy.device() == x.device(), "dy must have the shape and device of x [B, S, H, D]");
  c10::cuda::CUDAGuard g(x.device());
  const int64_t B = x.size(0), S = x.size(1), H = x.size(2), HD = x.size(3);
  TORCH_CHECK(HD == 128 || HD == 64, "head_dim must be 64 or 128");
  TORCH_CHECK(w.numel() == HD && w.device() == x.device(), "w must hold head_dim values on the device of x");
  check_f32(rstd, "rstd");
  TORCH_CHECK(rstd.numel() == B * S * H && rstd.device() == x.device(), "rstd must be [B, S, H] on the device of x");
  TORCH_CHECK(cosv.has_value() == sinv.has_value(), "cos and sin come together");
  if (cosv.has_value()) {
    check_f32(*cosv, "cos");
    check_f32(*sinv, "sin");
    TORCH_CHECK(cosv->dim() == 2 && cosv->size(0) == S && cosv->size(1) == HD / 2 && sinv->sizes() == cosv->sizes() &&
                    cosv->device() == x.device() && sinv->device() == x.device(), "cos/sin must be [S, D/2] on the device of x");
  }
  Tensor wf = w.to(at::kFloat).contiguous();
  const float* cp = cosv.has_value() ? cosv->data_ptr<float>() : nullptr;
  const float* sp = sinv.has_value() ? sinv->data_ptr<float>() : nullptr;
  Tensor dx = at::empty_like(x);
  Tensor dw = at::empty({HD}, x.options().dtype(at::kFloat));
  const int64_t blocks = cb200_rmsnorm_bwd_blocks(B * S * H, kRowsPerWarp);
  Tensor partials = at::empty({blocks, HD}, dw.options());
  cb200_rmsnorm_rope_bwd(dy.data_ptr(), x.data_ptr(), wf.data_ptr<float>(), rstd.data_ptr<float>(), cp, sp, dx.data_ptr(),
                         dw.data_ptr<float>(), partials.data_ptr<float>(), B * S * H, (int)S, (int)H, (int)HD, kRowsPerWarp,
                         stream());
  return {dx, dw};
}

Tensor gelu_fwd(const Tensor& x) {
  check_bf16(x, "x");
  TORCH_CHECK(x.numel() % 8 == 0, "numel must be a multiple of 8");
  c10::cuda::CUDAGuard g(x.device());
  Tensor y = at::empty_like(x);
  cb200_gelu_fwd(x.data_ptr(), y.data_ptr(), x.numel(), stream());
  return y;
}

Tensor gelu_bwd(const Tensor& dy, const Tensor& x) {
  check_bf16(x, "x");
  check_bf16(dy, "dy");
  c10::cuda::CUDAGuard g(x.device());
  Tensor dx = at::empty_like(x);
  cb200_gelu_bwd(dy.data_ptr(), x.data_ptr(), dx.data_ptr(), x.numel(), stream());
  return dx;
}

Tensor cfg_combine(const Tensor& c, const Tensor& u, double gval) {
  check_f32(c, "cond");
  check_f32(u, "uncond");
  c10::cuda::CUDAGuard g(c.device());
  Tensor o = at::empty_like(c);
  cb200_cfg_combine(c.data_ptr<float>(), u.data_ptr<float>(), o.data_ptr<float>(), (float)gval, c.numel(), stream());
  return o;
}

// out = sum_k coeffs[k] * xs[k]; fp32 tensors of one shape, at most 6
Tensor lincomb(at::TensorList xs, at::ArrayRef<double> coeffs) {
  TORCH_CHECK(!xs.empty() && xs.size() <= 6 && xs.size() == coeffs.size(), "lincomb takes 1 to 6 tensors and as many coefficients");
  const float* ptrs[6];
  float cs[6];
  for (size_t k = 0; k < xs.size(); ++k) {
    check_f32(xs[k], "operand");
    TORCH_CHECK(xs[k].sizes() == xs[0].sizes() && xs[k].device() == xs[0].device(), "lincomb operands differ in shape or device");
    TORCH_CHECK(reinterpret_cast<uintptr_t>(xs[k].data_ptr()) % 16 == 0, "lincomb operand is not 16-byte aligned");
    ptrs[k] = xs[k].data_ptr<float>();
    cs[k] = (float)coeffs[k];
  }
  c10::cuda::CUDAGuard g(xs[0].device());
  Tensor o = at::empty_like(xs[0]);
  TORCH_CHECK(cb200_lincomb(ptrs, cs, (int)xs.size(), o.data_ptr<float>(), o.numel(), stream()) == 0, "lincomb: bad operand count");
  return o;
}

// out = keep * mask + x * (1 - mask); keep = gt * flag[b] (noise absent) or noise - gt. x, gt, noise [B, C, ...] fp32, mask
// [B, 1, ...] fp32, flag [B] fp32.
Tensor frame_blend(const Tensor& x, const Tensor& gt, const c10::optional<Tensor>& noise, const Tensor& mask,
                   const c10::optional<Tensor>& flag, bool out_bf16) {
  check_f32(x, "x");
  check_f32(gt, "gt");
  check_f32(mask, "mask");
  TORCH_CHECK(x.dim() >= 3 && gt.sizes() == x.sizes(), "frame_blend: x and gt are [B, C, ...] of one shape");
  const long B = x.size(0), C = x.size(1), S = x.numel() / (B * C);
  TORCH_CHECK(mask.numel() == B * S, "frame_blend: the mask has one value per (sample, position)");
  if (noise.has_value()) {
    check_f32(*noise, "noise");
    TORCH_CHECK(noise->sizes() == x.sizes(), "frame_blend: noise and x differ in shape");
  }
  if (flag.has_value()) {
    check_f32(*flag, "flag");
    TORCH_CHECK(flag->numel() == B, "frame_blend: one flag per sample");
  }
  for (const Tensor* t : {&x, &gt, &mask, noise.has_value() ? &*noise : &x})
    TORCH_CHECK(reinterpret_cast<uintptr_t>(t->data_ptr()) % 16 == 0, "frame_blend operand is not 16-byte aligned");
  c10::cuda::CUDAGuard g(x.device());
  Tensor o = at::empty(x.sizes(), x.options().dtype(out_bf16 ? at::kBFloat16 : at::kFloat));
  TORCH_CHECK(cb200_frame_blend(x.data_ptr<float>(), gt.data_ptr<float>(), noise.has_value() ? noise->data_ptr<float>() : nullptr,
                                mask.data_ptr<float>(), flag.has_value() ? flag->data_ptr<float>() : nullptr, o.data_ptr(),
                                out_bf16 ? 1 : 0, B, C, S, stream()) == 0,
              "frame_blend: positions per channel must be a multiple of 4");
  return o;
}

void grad_cast_norm(const Tensor& g16, Tensor g32, Tensor sumsq, double scale) {
  check_bf16(g16, "grad");
  check_f32(g32, "grad_shard");
  check_f32(sumsq, "sumsq");
  TORCH_CHECK(g16.numel() == g32.numel(), "size mismatch");
  c10::cuda::CUDAGuard g(g16.device());
  Tensor partials = at::empty({cb200_grad_cast_norm_blocks(g16.numel())}, g32.options());
  cb200_grad_cast_norm(g16.data_ptr(), g32.data_ptr<float>(), sumsq.data_ptr<float>(), partials.data_ptr<float>(), (float)scale,
                       g16.numel(), stream());
}

void adamw_ema_shard(Tensor master, const Tensor& grad, Tensor m, Tensor v, const c10::optional<Tensor>& ema,
                     const c10::optional<Tensor>& out16, const Tensor& clip, double lr, double beta1, double beta2, double eps,
                     double wd, int64_t step, double ema_beta) {
  check_f32(master, "master");
  check_f32(grad, "grad");
  check_f32(m, "exp_avg");
  check_f32(v, "exp_avg_sq");
  check_f32(clip, "clip");
  c10::cuda::CUDAGuard g(master.device());
  float* ema_p = nullptr;
  void* out_p = nullptr;
  if (ema.has_value()) {
    check_f32(*ema, "ema");
    ema_p = ema->data_ptr<float>();
  }
  if (out16.has_value()) {
    check_bf16(*out16, "out16");
    TORCH_CHECK(out16->numel() >= master.numel(), "bf16 output too small");
    out_p = out16->data_ptr();
  }
  cb200_adamw_ema_shard(master.data_ptr<float>(), grad.data_ptr<float>(), m.data_ptr<float>(), v.data_ptr<float>(), ema_p, out_p,
                        clip.data_ptr<float>(), (float)lr, (float)beta1, (float)beta2, (float)eps, (float)wd, step,
                        (float)ema_beta, master.numel(), stream());
}

void cast_f32_bf16(const Tensor& src, Tensor dst) {
  check_f32(src, "src");
  check_bf16(dst, "dst");
  TORCH_CHECK(dst.numel() >= src.numel(), "dst too small");
  c10::cuda::CUDAGuard g(src.device());
  cb200_cast_f32_bf16(src.data_ptr<float>(), dst.data_ptr(), src.numel(), stream());
}

// ---- GEMM ------------------------------------------------------------------------------------
struct GemmDims {
  int M, N, K;
};

GemmDims gemm_dims(const Tensor& a, const Tensor& b, bool trans_a, bool trans_b) {
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2, "GEMM operands must be 2-D");
  GemmDims d;
  d.M = (int)(trans_a ? a.size(1) : a.size(0));
  d.K = (int)(trans_a ? a.size(0) : a.size(1));
  d.N = (int)(trans_b ? b.size(1) : b.size(0));
  const int64_t kb = trans_b ? b.size(0) : b.size(1);
  TORCH_CHECK(kb == d.K, "contraction dims differ: ", d.K, " vs ", kb);
  TORCH_CHECK(a.size(1) % 8 == 0 && b.size(1) % 8 == 0, "row strides must be multiples of 16 bytes");
  return d;
}

int sm_count(int device) {
  static int cache[64] = {0};
  if (cache[device] == 0) cache[device] = at::cuda::getDeviceProperties(device)->multiProcessorCount;
  return cache[device];
}

Tensor gemm_impl(const Tensor& a, const Tensor& b, const c10::optional<Tensor>& bias, int64_t act, bool trans_a, bool trans_b,
                 Tensor* pre, const Tensor* resid, const Tensor* gate, int64_t L) {
  check_bf16(a, "a");
  check_bf16(b, "b");
  c10::cuda::CUDAGuard g(a.device());
  const GemmDims d = gemm_dims(a, b, trans_a, trans_b);
  Tensor c = at::empty({d.M, d.N}, a.options());
  const void* bias_p = nullptr;
  Tensor bias_c;
  if (bias.has_value()) {
    bias_c = bias->to(at::kBFloat16).contiguous();
    TORCH_CHECK(bias_c.numel() == d.N, "bias must be [N]");
    bias_p = bias_c.data_ptr();
  }
  void* pre_p = nullptr;
  if (pre != nullptr) {
    *pre = at::empty({d.M, d.N}, a.options());
    pre_p = pre->data_ptr();
  }
  const void* resid_p = nullptr;
  const float* gate_p = nullptr;
  if (resid != nullptr) {
    check_bf16(*resid, "resid");
    check_f32(*gate, "gate");
    TORCH_CHECK(resid->numel() == (int64_t)d.M * d.N && gate->size(-1) == d.N && gate->numel() == (d.M / L) * (int64_t)d.N,
                "gated-residual epilogue shapes");
    resid_p = resid->data_ptr();
    gate_p = gate->data_ptr<float>();
  }
  const int dev = a.get_device();
  const int rc = cb200_gemm_bf16(a.data_ptr(), b.data_ptr(), c.data_ptr(), d.M, d.N, d.K, trans_a ? 1 : 0, trans_b ? 1 : 0, bias_p,
                                 (int)act, pre_p, resid_p, gate_p, (int)L, error_word(dev), sm_count(dev), stream());
  TORCH_CHECK(rc == 0, "tcgen05 GEMM launch failed with code ", rc);
  return c;
}

Tensor gemm_bf16(const Tensor& a, const Tensor& b, const c10::optional<Tensor>& bias, int64_t act, bool trans_a, bool trans_b) {
  return gemm_impl(a, b, bias, act, trans_a, trans_b, nullptr, nullptr, nullptr, 1);
}

std::tuple<Tensor, Tensor> gemm_bf16_gelu_pre(const Tensor& a, const Tensor& b, const c10::optional<Tensor>& bias) {
  Tensor pre;
  Tensor c = gemm_impl(a, b, bias, 1, false, false, &pre, nullptr, nullptr, 1);
  return {c, pre};
}

// resid + gate * (a @ b^T) and, as a second output, the product itself (training keeps it for the gate gradient)
std::tuple<Tensor, Tensor> gemm_bf16_gate_residual_pre(const Tensor& a, const Tensor& b, const Tensor& resid, const Tensor& gate,
                                                       int64_t L) {
  TORCH_CHECK(b.size(0) % 256 == 0, "the two-output gated-residual epilogue needs whole 256-column tiles");
  Tensor pre;
  Tensor c = gemm_impl(a, b, c10::nullopt, 0, false, false, &pre, &resid, &gate, L);
  return {c, pre};
}

Tensor gemm_bf16_gate_residual(const Tensor& a, const Tensor& b, const Tensor& resid, const Tensor& gate, int64_t L) {
  return gemm_impl(a, b, c10::nullopt, 0, false, false, nullptr, &resid, &gate, L);
}

// x [B*S, K] @ w [H*128, K]^T with the Ulysses sequence->head exchange as the epilogue: nothing is returned, head h of token
// (b, s) lands in out_ptrs[h / (H/P)] (a staging buffer of that rank, [B, P*S, H/P, 128]) after optional RMSNorm and RoPE.
// ``keep_raw`` (training; needs norm_w): also returns the un-normalised projection [B*S, H*128] and the reciprocal RMS [B*S, H]
// that the RMSNorm backward needs; otherwise two empty tensors.
std::tuple<Tensor, Tensor> gemm_scatter_heads_peer(const Tensor& x, const Tensor& w, c10::ArrayRef<int64_t> out_ptrs,
                                                   const c10::optional<Tensor>& norm_w, const c10::optional<Tensor>& cosv,
                                                   const c10::optional<Tensor>& sinv, int64_t S, int64_t rank, double eps,
                                                   bool keep_raw) {
  check_bf16(x, "x");
  check_bf16(w, "w");
  TORCH_CHECK(x.is_contiguous() && w.is_contiguous(), "operands must be contiguous");
  c10::cuda::CUDAGuard g(x.device());
  const GemmDims d = gemm_dims(x, w, false, false);
  TORCH_CHECK(d.N % 128 == 0 && out_ptrs.size() >= 1 && out_ptrs.size() <= 8 && (d.N / 128) % (int64_t)out_ptrs.size() == 0,
              "heads of 128 channels, divisible by the peer count");
  TORCH_CHECK(S > 0 && d.M % S == 0, "rows must be B * S");
  Tensor wf;
  const float *wp = nullptr, *cp = nullptr, *sp = nullptr;
  if (norm_w.has_value()) {
    wf = norm_w->to(at::kFloat).contiguous();
    TORCH_CHECK(wf.numel() == 128, "norm weight must be [128]");
    wp = wf.data_ptr<float>();
    if (cosv.has_value()) {
      check_f32(*cosv, "cos");
      check_f32(*sinv, "sin");
      TORCH_CHECK(cosv->numel() >= S * 64 && sinv->numel() >= S * 64 && cosv->is_contiguous() && sinv->is_contiguous(),
                  "cos/sin must be [S, 64]");
      cp = cosv->data_ptr<float>();
      sp = sinv->data_ptr<float>();
    }
  }
  TORCH_CHECK(rank >= 0 && rank < (int64_t)out_ptrs.size(), "rank out of range");
  TORCH_CHECK(!keep_raw || wp != nullptr, "keep_raw needs a norm weight (without normalisation the output is the raw projection)");
  Tensor raw = at::empty({keep_raw ? (int64_t)d.M : 0, keep_raw ? (int64_t)d.N : 0}, x.options());
  Tensor rstd = at::empty({keep_raw ? (int64_t)d.M : 0, keep_raw ? (int64_t)d.N / 128 : 0}, x.options().dtype(at::kFloat));
  std::vector<int64_t> p(out_ptrs.begin(), out_ptrs.end());
  const int dev = x.get_device();
  const int rc = cb200_gemm_bf16_scatter_heads(x.data_ptr(), w.data_ptr(), d.M, d.N, d.K, p.data(), (int)p.size(), (int)rank, (int)S,
                                               wp, cp, sp, (float)eps, keep_raw ? raw.data_ptr() : nullptr,
                                               keep_raw ? rstd.data_ptr<float>() : nullptr, error_word(dev), sm_count(dev), stream());
  TORCH_CHECK(rc == 0, "tcgen05 GEMM (head-scatter epilogue) launch failed with code ", rc);
  return {raw, rstd};
}

std::tuple<Tensor, Tensor> ln_modulate_jvp(const Tensor& x, const Tensor& tx, const Tensor& shift, const Tensor& scale,
                                           const c10::optional<Tensor>& tshift, const c10::optional<Tensor>& tscale, int64_t L,
                                           double eps) {
  check_bf16(x, "x");
  check_bf16(tx, "tx");
  check_f32(shift, "shift");
  check_f32(scale, "scale");
  TORCH_CHECK(x.dim() == 2 && tx.sizes() == x.sizes() && tx.device() == x.device(), "tx must have the shape and device of x [rows, D]");
  c10::cuda::CUDAGuard g(x.device());
  const int64_t rows = x.size(0), D = x.size(1);
  TORCH_CHECK(D % 8 == 0 && D <= 8192, "channel dim must be a multiple of 8 and <= 8192");
  TORCH_CHECK(L > 0 && rows % L == 0 && shift.dim() == 2 && shift.size(0) == rows / L && shift.size(1) == D &&
                  scale.sizes() == shift.sizes(), "shift/scale must be [rows/L, D]");
  TORCH_CHECK(tshift.has_value() == tscale.has_value(), "give both modulation tangents or neither");
  const float* tsp = nullptr;
  const float* tcp = nullptr;
  if (tshift.has_value()) {
    check_f32(*tshift, "tshift");
    check_f32(*tscale, "tscale");
    TORCH_CHECK(tshift->sizes() == shift.sizes() && tscale->sizes() == shift.sizes(), "modulation tangents must be [rows/L, D]");
    tsp = tshift->data_ptr<float>();
    tcp = tscale->data_ptr<float>();
  }
  // value and tangent rows in one allocation, tangent after value: a following GEMM can take both as one [2 rows, D] operand
  Tensor both = at::empty({2, rows, D}, x.options());
  Tensor y = both.select(0, 0), ty = both.select(0, 1);
  cb200_ln_modulate_jvp(x.data_ptr(), tx.data_ptr(), shift.data_ptr<float>(), scale.data_ptr<float>(), tsp, tcp, y.data_ptr(),
                        ty.data_ptr(), rows, (int)D, (int)L, (float)eps, stream());
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return {y, ty};
}

std::tuple<Tensor, Tensor> rmsnorm_rope_jvp(const Tensor& x, const Tensor& tx, const Tensor& w, const c10::optional<Tensor>& cosv,
                                            const c10::optional<Tensor>& sinv, double eps) {
  check_bf16(x, "x");
  check_bf16(tx, "tx");
  TORCH_CHECK(x.dim() == 4 && tx.sizes() == x.sizes() && tx.device() == x.device(), "tx must have the shape and device of x [B, S, H, D]");
  c10::cuda::CUDAGuard g(x.device());
  const int64_t B = x.size(0), S = x.size(1), H = x.size(2), HD = x.size(3);
  TORCH_CHECK(HD == 128 || HD == 64, "head_dim must be 64 or 128");
  TORCH_CHECK(w.numel() == HD && w.device() == x.device(), "w must hold head_dim values on the device of x");
  Tensor wf = w.to(at::kFloat).contiguous();
  const float* cp = nullptr;
  const float* sp = nullptr;
  TORCH_CHECK(cosv.has_value() == sinv.has_value(), "give both rotation tables or neither");
  if (cosv.has_value()) {
    check_f32(*cosv, "cos");
    check_f32(*sinv, "sin");
    TORCH_CHECK(cosv->dim() == 2 && cosv->size(0) == S && cosv->size(1) == HD / 2 && sinv->sizes() == cosv->sizes(),
                "cos/sin must be [S, D/2]");
    cp = cosv->data_ptr<float>();
    sp = sinv->data_ptr<float>();
  }
  Tensor y = at::empty_like(x), ty = at::empty_like(x);
  cb200_rmsnorm_rope_jvp(x.data_ptr(), tx.data_ptr(), wf.data_ptr<float>(), cp, sp, y.data_ptr(), ty.data_ptr(), B * S * H, (int)S,
                         (int)H, (int)HD, (float)eps, stream());
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return {y, ty};
}

// Z small fp32 GEMMs in one launch (skinny.cu). ``a``: fp32 storage addressed as a[z*a_z + r*a_r + k*a_k]; B: either ``b_ptrs``
// (int64 device tensor with one base address per problem) or the tensor ``b`` addressed as b[z*b_z + n*b_n + k*b_k], bf16 or
// fp32; result [Z, R, N] contiguous in ``out_bf16 ? bf16 : fp32``; with ``ksplit`` > 1 the result is [Z * ksplit, R, N] fp32:
// partial sums over ``ksplit`` ranges of k, to be added by the caller (few tiles, long reduction: more CTAs in flight).
Tensor skinny_bgemm(const Tensor& a, int64_t a_z, int64_t a_r, int64_t a_k, const c10::optional<Tensor>& b_ptrs,
                    const c10::optional<Tensor>& b, int64_t b_z, int64_t b_n, int64_t b_k, bool b_bf16,
                    const c10::optional<Tensor>& add, int64_t add_cols, int64_t Z, int64_t R, int64_t N, int64_t K, bool silu_a,
                    bool silu_b, bool out_bf16, int64_t ksplit) {
  check_f32(a, "a");
  c10::cuda::CUDAGuard g(a.device());
  TORCH_CHECK(Z > 0 && R > 0 && N > 0 && K > 0 && ksplit >= 1 && Z * ksplit <= 65535, "skinny_bgemm: bad problem size");
  TORCH_CHECK(ksplit == 1 || !out_bf16, "skinny_bgemm: partial sums (ksplit > 1) are fp32");
  TORCH_CHECK(a_z >= 0 && a_r >= 0 && a_k >= 0 && b_z >= 0 && b_n >= 0 && b_k >= 0, "skinny_bgemm: strides must not be negative");
  TORCH_CHECK((Z - 1) * a_z + (R - 1) * a_r + (K - 1) * a_k < a.numel(), "skinny_bgemm: A strides reach past the tensor");
  TORCH_CHECK(b_ptrs.has_value() != b.has_value(), "skinny_bgemm: give exactly one of b_ptrs and b");
  const long long* bp = nullptr;
  const void* bb = nullptr;
  if (b_ptrs.has_value()) {
    TORCH_CHECK(b_ptrs->is_cuda() && b_ptrs->scalar_type() == at::kLong && b_ptrs->is_contiguous() && b_ptrs->numel() >= Z,
                "b_ptrs must be a contiguous int64 CUDA tensor with one entry per problem");
    bp = reinterpret_cast<const long long*>(b_ptrs->data_ptr<int64_t>());
  } else {
    TORCH_CHECK(b->is_cuda() && b->is_contiguous() && b->scalar_type() == (b_bf16 ? at::kBFloat16 : at::kFloat),
                "b must be a contiguous CUDA tensor of the stated dtype");
    TORCH_CHECK((Z - 1) * b_z + (N - 1) * b_n + (K - 1) * b_k < b->numel(), "skinny_bgemm: B strides reach past the tensor");
    bb = b->data_ptr();
  }
  const float* addp = nullptr;
  int ld_add = 0;
  if (add.has_value()) {
    check_f32(*add, "add");
    TORCH_CHECK(add->dim() == 2 && add->size(0) == R && add_cols >= 0 && add_cols <= add->size(1) && add_cols <= N,
                "add must be [R, >= add_cols] with add_cols <= N");
    addp = add->data_ptr<float>();
    ld_add = (int)add->size(1);
  }
  Tensor c = at::empty({Z * ksplit, R, N}, a.options().dtype(out_bf16 ? at::kBFloat16 : at::kFloat));
  const int rc = cb200_skinny_bgemm(a.data_ptr<float>(), a_z, a_r, a_k, bp, bb, b_z, b_n, b_k, b_bf16 ? 1 : 0, c.data_ptr(), R * N,
                                    (int)N, out_bf16 ? 1 : 0, addp, ld_add, (int)add_cols, (int)Z, (int)R, (int)N, (int)K,
                                    silu_a ? 1 : 0, silu_b ? 1 : 0, (int)ksplit, stream());
  TORCH_CHECK(rc == 0, "skinny_bgemm launch refused with code ", rc);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return c;
}

// tile mode of the GEMM: 0 single-CTA 128 x 256 tiles, 1 CTA pairs (256 x 256 per pair), -1 only reads; returns the previous mode
int64_t gemm_pair_mode(int64_t mode) { return cb200_gemm_pair_mode((int)mode); }

int64_t kernel_error(int64_t device, bool clear) {
  int v = 0;
  int* w = error_word((int)device);
  C10_CUDA_CHECK(cudaMemcpy(&v, w, sizeof(int), cudaMemcpyDeviceToHost));
  if (clear && v != 0) C10_CUDA_CHECK(cudaMemset(w, 0, sizeof(int)));
  return v;
}

}  // namespace

// defined in bindings_attn.cpp / bindings_peer.cpp
void register_attention_ops(torch::Library& m);
void register_peer_ops(torch::Library& m);
void register_conv_ops(torch::Library& m);

TORCH_LIBRARY(cosmos_b200, m) {
  m.def("ln_modulate_fwd(Tensor x, Tensor shift, Tensor scale, int L, float eps) -> (Tensor, Tensor, Tensor)", &ln_modulate_fwd);
  m.def("ln_modulate_bwd(Tensor dy, Tensor x, Tensor mean, Tensor rstd, Tensor scale, int L) -> (Tensor, Tensor, Tensor)",
        &ln_modulate_bwd);
  m.def("gate_residual_fwd(Tensor x, Tensor gate, Tensor y, int L) -> Tensor", &gate_residual_fwd);
  m.def("gate_residual_bwd(Tensor dout, Tensor gate, Tensor y, int L) -> (Tensor, Tensor)", &gate_residual_bwd);
  m.def("rmsnorm_rope_fwd(Tensor x, Tensor w, Tensor? cos, Tensor? sin, float eps) -> (Tensor, Tensor)", &rmsnorm_rope_fwd);
  m.def("rmsnorm_rope_bwd(Tensor dy, Tensor x, Tensor w, Tensor rstd, Tensor? cos, Tensor? sin) -> (Tensor, Tensor)",
        &rmsnorm_rope_bwd);
  m.def("gelu_fwd(Tensor x) -> Tensor", &gelu_fwd);
  m.def("gelu_bwd(Tensor dy, Tensor x) -> Tensor", &gelu_bwd);
  m.def("cfg_combine(Tensor cond, Tensor uncond, float guidance) -> Tensor", &cfg_combine);
  m.def("lincomb(Tensor[] xs, float[] coeffs) -> Tensor", &lincomb);
  m.def("frame_blend(Tensor x, Tensor gt, Tensor? noise, Tensor mask, Tensor? flag, bool out_bf16) -> Tensor", &frame_blend);
  m.def("grad_cast_norm(Tensor g16, Tensor(a!) g32, Tensor(b!) sumsq, float scale) -> ()", &grad_cast_norm);
  m.def("adamw_ema_shard(Tensor(a!) master, Tensor grad, Tensor(b!) m, Tensor(c!) v, Tensor(d!)? ema, Tensor(e!)? out16, "
        "Tensor clip, float lr, float beta1, float beta2, float eps, float wd, int step, float ema_beta) -> ()",
        &adamw_ema_shard);
  m.def("cast_f32_bf16(Tensor src, Tensor(a!) dst) -> ()", &cast_f32_bf16);
  // schema only; kernels sit under the CUDA key (end of file) so dispatch modes can intercept them
  m.def("gemm_bf16(Tensor a, Tensor b, Tensor? bias, int act, bool trans_a, bool trans_b) -> Tensor");
  m.def("gemm_bf16_gelu_pre(Tensor a, Tensor b, Tensor? bias) -> (Tensor, Tensor)");
  m.def("gemm_bf16_gate_residual(Tensor a, Tensor b, Tensor resid, Tensor gate, int L) -> Tensor");
  m.def("gemm_bf16_gate_residual_pre(Tensor a, Tensor b, Tensor resid, Tensor gate, int L) -> (Tensor, Tensor)");
  m.def("gemm_scatter_heads_peer(Tensor x, Tensor w, int[] out_ptrs, Tensor? norm_w, Tensor? cos, Tensor? sin, int S, int rank, "
        "float eps, bool keep_raw) -> (Tensor, Tensor)", &gemm_scatter_heads_peer);
  m.def("ln_modulate_jvp(Tensor x, Tensor tx, Tensor shift, Tensor scale, Tensor? tshift, Tensor? tscale, int L, float eps) -> "
        "(Tensor, Tensor)", &ln_modulate_jvp);
  m.def("rmsnorm_rope_jvp(Tensor x, Tensor tx, Tensor w, Tensor? cos, Tensor? sin, float eps) -> (Tensor, Tensor)", &rmsnorm_rope_jvp);
  m.def("skinny_bgemm(Tensor a, int a_z, int a_r, int a_k, Tensor? b_ptrs, Tensor? b, int b_z, int b_n, int b_k, bool b_bf16, "
        "Tensor? add, int add_cols, int Z, int R, int N, int K, bool silu_a, bool silu_b, bool out_bf16, int ksplit) -> Tensor", &skinny_bgemm);
  m.def("gemm_pair_mode(int mode) -> int", &gemm_pair_mode);
  m.def("kernel_error(int device, bool clear) -> int", &kernel_error);
  register_attention_ops(m);
  register_peer_ops(m);
  register_conv_ops(m);
}

TORCH_LIBRARY_IMPL(cosmos_b200, CUDA, m) {
  m.impl("gemm_bf16", &gemm_bf16);
  m.impl("gemm_bf16_gelu_pre", &gemm_bf16_gelu_pre);
  m.impl("gemm_bf16_gate_residual", &gemm_bf16_gate_residual);
  m.impl("gemm_bf16_gate_residual_pre", &gemm_bf16_gate_residual_pre);
}
