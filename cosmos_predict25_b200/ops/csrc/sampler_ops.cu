// Element-wise kernels of the sampling loop (one pass over memory each, fp32 math, 16-byte accesses):
//
//   lincomb       out = sum_k c_k * x_k, up to 6 fp32 operands: every state update of the multistep solver (data prediction,
//                 predictor, corrector) is one launch instead of 2 - 9 torch kernels that each re-read the state
//   frame_blend   out = keep * m + x * (1 - m) with the frame mask broadcast over channels; keep = gt * flag[b] (conditioning
//                 frames put back into the noisy latent) or keep = noise - gt (their velocity put back into the network output);
//                 optional bf16 output, so the cast to the network's dtype costs no extra pass
//
// Reference behaviour these restate: the scheduler's tensor arithmetic (diffusers-style UniPC in
// cosmos_predict2/_src/predict2/schedulers) and the replacement of conditioning frames in
// cosmos_predict2/_src/predict2/models/video2world_model_rectified_flow.py (denoise).

#include "common.cuh"
#include "launchers.h"

namespace cb200 {

constexpr int kLcMax = 6;
struct LincombArgs {
  const float* x[kLcMax];
  float c[kLcMax];
};

template <int N>
__global__ void __launch_bounds__(256) lincomb_kernel(LincombArgs a, float* __restrict__ out, long n) {
  const long nvec = n >> 2;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long)gridDim.x * blockDim.x) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int k = 0; k < N; ++k) {
      const float4 v = reinterpret_cast<const float4*>(a.x[k])[i];
      acc.x = fmaf(a.c[k], v.x, acc.x);
      acc.y = fmaf(a.c[k], v.y, acc.y);
      acc.z = fmaf(a.c[k], v.z, acc.z);
      acc.w = fmaf(a.c[k], v.w, acc.w);
    }
    reinterpret_cast<float4*>(out)[i] = acc;
  }
  if (blockIdx.x == 0) {
    for (long i = (nvec << 2) + threadIdx.x; i < n; i += blockDim.x) {
      float acc = 0.f;
#pragma unroll
      for (int k = 0; k < N; ++k) acc = fmaf(a.c[k], a.x[k][i], acc);
      out[i] = acc;
    }
  }
}

// x, gt, noise: [B, C, S] fp32 (S = frames x rows x columns); mask: [B, S] fp32 (one value per position, shared by the channels);
// flag: [B] fp32 or null (1); noise null: keep = gt * flag, else keep = noise - gt. OUT_BF16: out is bf16.
template <bool OUT_BF16>
__global__ void __launch_bounds__(256) frame_blend_kernel(const float* __restrict__ x, const float* __restrict__ gt,
                                                          const float* __restrict__ noise, const float* __restrict__ mask,
                                                          const float* __restrict__ flag, void* __restrict__ out, long C, long S,
                                                          long n) {
  // S % 4 == 0 is checked by the launcher: a 4-vector never crosses a channel row
  const long nvec = n >> 2, svec = S >> 2;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long)gridDim.x * blockDim.x) {
    const long row = i / svec, s4 = i - row * svec, b = row / C;
    const float4 m = reinterpret_cast<const float4*>(mask)[b * svec + s4];
    const float4 xv = reinterpret_cast<const float4*>(x)[i];
    float4 g = reinterpret_cast<const float4*>(gt)[i];
    if (noise != nullptr) {
      const float4 z = reinterpret_cast<const float4*>(noise)[i];
      g = make_float4(z.x - g.x, z.y - g.y, z.z - g.z, z.w - g.w);
    } else if (flag != nullptr) {
      const float f = flag[b];
      g = make_float4(g.x * f, g.y * f, g.z * f, g.w * f);
    }
    float4 o;
    o.x = fmaf(g.x, m.x, xv.x * (1.f - m.x));
    o.y = fmaf(g.y, m.y, xv.y * (1.f - m.y));
    o.z = fmaf(g.z, m.z, xv.z * (1.f - m.z));
    o.w = fmaf(g.w, m.w, xv.w * (1.f - m.w));
    if (OUT_BF16) {
      __nv_bfloat162 lo = __floats2bfloat162_rn(o.x, o.y), hi = __floats2bfloat162_rn(o.z, o.w);
      uint2 pk;
      pk.x = *reinterpret_cast<uint32_t*>(&lo);
      pk.y = *reinterpret_cast<uint32_t*>(&hi);
      reinterpret_cast<uint2*>(out)[i] = pk;
    } else {
      reinterpret_cast<float4*>(out)[i] = o;
    }
  }
}

static int grid_for(long work_items) {
  long blocks = (work_items + 255) / 256;
  const long cap = 148L * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (int)blocks;
}

}  // namespace cb200

int cb200_lincomb(const float* const* xs, const float* cs, int count, float* out, long n, cudaStream_t st) {
  using namespace cb200;
  if (count < 1 || count > kLcMax) return 1;
  LincombArgs a;
  for (int k = 0; k < kLcMax; ++k) {
    a.x[k] = k < count ? xs[k] : nullptr;
    a.c[k] = k < count ? cs[k] : 0.f;
  }
  const int grid = grid_for(n >> 2);
  switch (count) {
    case 1: lincomb_kernel<1><<<grid, 256, 0, st>>>(a, out, n); break;
    case 2: lincomb_kernel<2><<<grid, 256, 0, st>>>(a, out, n); break;
    case 3: lincomb_kernel<3><<<grid, 256, 0, st>>>(a, out, n); break;
    case 4: lincomb_kernel<4><<<grid, 256, 0, st>>>(a, out, n); break;
    case 5: lincomb_kernel<5><<<grid, 256, 0, st>>>(a, out, n); break;
    default: lincomb_kernel<6><<<grid, 256, 0, st>>>(a, out, n); break;
  }
  return 0;
}

int cb200_frame_blend(const float* x, const float* gt, const float* noise, const float* mask, const float* flag, void* out,
                      int out_bf16, long B, long C, long S, cudaStream_t st) {
  using namespace cb200;
  if (S % 4 != 0) return 1;
  const long n = B * C * S;
  const int grid = grid_for(n >> 2);
  if (out_bf16)
    frame_blend_kernel<true><<<grid, 256, 0, st>>>(x, gt, noise, mask, flag, out, C, S, n);
  else
    frame_blend_kernel<false><<<grid, 256, 0, st>>>(x, gt, noise, mask, flag, out, C, S, n);
  return 0;
}
