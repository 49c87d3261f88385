// Forward-mode (tangent) variants of the DiT block's element-wise kernels: value and directional derivative in one pass over the
// row. Used by the network JVP of the consistency-distillation step (student value and d/dt along the teacher ODE), where the
// attention runs on fa_jvp.cu and the GEMMs take primal and tangent rows in one call.
//
//   ln_modulate_jvp     y  = xhat (1 + scale) + shift,                 xhat = (x - mean) rstd
//                       ty = txhat (1 + scale) + xhat tscale + tshift, txhat = rstd ((tx - mean(tx)) - xhat mean(xhat (tx - mean(tx))))
//   rmsnorm_rope_jvp    n  = w x rstd,  tn = w (tx rstd - x rstd^3 mean(x tx)),  then the same rotation on both (it is linear)

#include "common.cuh"
#include "launchers.h"

namespace cb200 {

constexpr int kTanThreads = 256;

__device__ __forceinline__ void tan_load_f8(const float* p, float (&f)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p);
  const float4 b = *reinterpret_cast<const float4*>(p + 4);
  f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w;
  f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}

// one CTA per token row; tshift / tscale may be null (no tangent on the modulation)
template <int MV>
__global__ void __launch_bounds__(kTanThreads) ln_modulate_jvp_kernel(
    const bf16* __restrict__ x, const bf16* __restrict__ tx, const float* __restrict__ shift, const float* __restrict__ scale,
    const float* __restrict__ tshift, const float* __restrict__ tscale, bf16* __restrict__ y, bf16* __restrict__ ty, int D, int L,
    float eps) {
  __shared__ float red[64];
  const long row = blockIdx.x;
  const long frame = row / L;
  const int nvec = D >> 3;
  const bf16x8* xr = reinterpret_cast<const bf16x8*>(x + row * D);
  const bf16x8* tr = reinterpret_cast<const bf16x8*>(tx + row * D);
  float v[MV][8], t[MV][8];
  float s = 0.f, st = 0.f;
#pragma unroll
  for (int i = 0; i < MV; ++i) {
    const int c = threadIdx.x + i * kTanThreads;
    if (c < nvec) {
      unpack8(xr[c], v[i]);
      unpack8(tr[c], t[i]);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        s += v[i][j];
        st += t[i][j];
      }
    }
  }
  const float mean = block_sum(s, red) / D;
  const float tmean = block_sum(st, red) / D;
  float q = 0.f, cx = 0.f;
#pragma unroll
  for (int i = 0; i < MV; ++i) {
    const int c = threadIdx.x + i * kTanThreads;
    if (c < nvec) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float d = v[i][j] - mean;
        q += d * d;
        cx += d * (t[i][j] - tmean);
      }
    }
  }
  const float rstd = rsqrtf(block_sum(q, red) / D + eps);
  const float cross = block_sum(cx, red) / D * rstd;      // mean(xhat (tx - tmean))
  bf16x8* yr = reinterpret_cast<bf16x8*>(y + row * D);
  bf16x8* tyr = reinterpret_cast<bf16x8*>(ty + row * D);
#pragma unroll
  for (int i = 0; i < MV; ++i) {
    const int c = threadIdx.x + i * kTanThreads;
    if (c < nvec) {
      float a[8], b[8], ta[8], tb[8], o[8], to[8];
      tan_load_f8(shift + frame * D + c * 8, a);
      tan_load_f8(scale + frame * D + c * 8, b);
      if (tshift != nullptr) {
        tan_load_f8(tshift + frame * D + c * 8, ta);
        tan_load_f8(tscale + frame * D + c * 8, tb);
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) ta[j] = tb[j] = 0.f;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float xh = (v[i][j] - mean) * rstd;
        const float txh = rstd * ((t[i][j] - tmean) - xh * cross);
        o[j] = xh * (1.f + b[j]) + a[j];
        to[j] = txh * (1.f + b[j]) + xh * tb[j] + ta[j];
      }
      yr[c] = pack8(o);
      tyr[c] = pack8(to);
    }
  }
}

// one warp per (token, head); head_dim in {64, 128}
template <int HD>
__global__ void __launch_bounds__(256) rmsnorm_rope_jvp_kernel(
    const bf16* __restrict__ x, const bf16* __restrict__ tx, const float* __restrict__ w, const float* __restrict__ cosv,
    const float* __restrict__ sinv, bf16* __restrict__ y, bf16* __restrict__ ty, long n_rows, int S, int H, float eps) {
  constexpr int E = HD / 32;
  const int lane = threadIdx.x & 31;
  const long row = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= n_rows) return;
  const long s = (row / H) % S;
  float v[E], t[E];
#pragma unroll
  for (int j = 0; j < E; j += 2) {
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(x + row * HD + lane * E + j));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(tx + row * HD + lane * E + j));
    v[j] = a.x; v[j + 1] = a.y;
    t[j] = b.x; t[j + 1] = b.y;
  }
  float ss = 0.f, cx = 0.f;
#pragma unroll
  for (int j = 0; j < E; ++j) {
    ss += v[j] * v[j];
    cx += v[j] * t[j];
  }
  ss = warp_sum(ss);
  cx = warp_sum(cx);
  const float rstd = rsqrtf(ss / HD + eps);
  const float k = rstd * rstd * rstd * (cx / HD);
  float o[E], to[E];
#pragma unroll
  for (int j = 0; j < E; ++j) {
    const float wj = w[lane * E + j];
    o[j] = v[j] * rstd * wj;
    to[j] = (t[j] * rstd - v[j] * k) * wj;
  }
  if (cosv != nullptr) {
    const int half_idx = (lane & 15) * E;
#pragma unroll
    for (int j = 0; j < E; ++j) {
      const float other = __shfl_xor_sync(0xffffffffu, o[j], 16);
      const float tother = __shfl_xor_sync(0xffffffffu, to[j], 16);
      const float c = cosv[s * (HD / 2) + half_idx + j];
      const float sn = sinv[s * (HD / 2) + half_idx + j];
      o[j] = (lane < 16) ? (o[j] * c - other * sn) : (o[j] * c + other * sn);
      to[j] = (lane < 16) ? (to[j] * c - tother * sn) : (to[j] * c + tother * sn);
    }
  }
#pragma unroll
  for (int j = 0; j < E; j += 2) {
    *reinterpret_cast<__nv_bfloat162*>(y + row * HD + lane * E + j) = __floats2bfloat162_rn(o[j], o[j + 1]);
    *reinterpret_cast<__nv_bfloat162*>(ty + row * HD + lane * E + j) = __floats2bfloat162_rn(to[j], to[j + 1]);
  }
}

}  // namespace cb200

using namespace cb200;

extern "C" {

void cb200_ln_modulate_jvp(const void* x, const void* tx, const float* shift, const float* scale, const float* tshift,
                           const float* tscale, void* y, void* ty, long rows, int D, int L, float eps, cudaStream_t st) {
#define LAUNCH(MV)                                                                                                              \
  ln_modulate_jvp_kernel<MV><<<(unsigned)rows, kTanThreads, 0, st>>>((const bf16*)x, (const bf16*)tx, shift, scale, tshift, tscale, \
                                                                     (bf16*)y, (bf16*)ty, D, L, eps)
  if (D <= 2048) LAUNCH(1); else if (D <= 4096) LAUNCH(2); else LAUNCH(4);
#undef LAUNCH
}

void cb200_rmsnorm_rope_jvp(const void* x, const void* tx, const float* w, const float* cosv, const float* sinv, void* y, void* ty,
                            long n_rows, int S, int H, int HD, float eps, cudaStream_t st) {
  const unsigned blocks = (unsigned)((n_rows + 7) / 8);
  if (HD == 128)
    rmsnorm_rope_jvp_kernel<128><<<blocks, 256, 0, st>>>((const bf16*)x, (const bf16*)tx, w, cosv, sinv, (bf16*)y, (bf16*)ty, n_rows,
                                                         S, H, eps);
  else
    rmsnorm_rope_jvp_kernel<64><<<blocks, 256, 0, st>>>((const bf16*)x, (const bf16*)tx, w, cosv, sinv, (bf16*)y, (bf16*)ty, n_rows,
                                                        S, H, eps);
}

}  // extern "C"
