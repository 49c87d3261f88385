// Memory-bound fused kernels of the DiT block and of the optimizer (sm_100a).
//
//   ln_modulate      LayerNorm(no affine) * (1 + scale[frame]) + shift[frame]       fwd + bwd
//   gate_residual    x + gate[frame] * y                                             fwd + bwd
//   rmsnorm_rope     per-head RMSNorm (learnable weight) + rotate-half RoPE          fwd + bwd
//   gelu             exact (erf) GELU                                                fwd + bwd
//   cfg_combine      cond + g * (cond - uncond)
//   grad_cast_norm   bf16 grad -> fp32 * scale, NaN/Inf scrub, squared-norm partials
//   adamw_ema_shard  AdamW on fp32 masters + EMA + bf16 write-back, clip coefficient read on device
//
// Every kernel moves each byte once: 16-byte vector accesses, fp32 math in registers, one pass.
// Reductions over tokens (dshift/dscale/dgate/dweight) are two-stage and deterministic: per-CTA
// partials go to a scratch buffer, a second kernel sums them in a fixed order.

#include "common.cuh"
#include "launchers.h"
#include "sm100.cuh"   // packed fp32x2 arithmetic

namespace cb200 {
using sm100::add2;
using sm100::fma2;
using sm100::mul2;

// element pair i of an 8-value register row
#define CB200_P2(arr, i) make_float2((arr)[2 * (i)], (arr)[2 * (i) + 1])

constexpr int kThreads = 256;
constexpr int kMaxVec = 4;  // up to 256*4*8 = 8192 channels per row

__device__ __forceinline__ float2 block_sum2(float a, float b, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  a = warp_sum(a);
  b = warp_sum(b);
  __syncthreads();
  if (lane == 0) {
    red[warp] = a;
    red[32 + warp] = b;
  }
  __syncthreads();
  const int nwarps = (blockDim.x + 31) >> 5;
  float ta = (lane < nwarps) ? red[lane] : 0.f;
  float tb = (lane < nwarps) ? red[32 + lane] : 0.f;
  return make_float2(warp_sum(ta), warp_sum(tb));
}

__device__ __forceinline__ void load_f8(const float* p, float (&f)[8]) {
  float4 a = *reinterpret_cast<const float4*>(p);
  float4 b = *reinterpret_cast<const float4*>(p + 4);
  f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w;
  f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}

__device__ __forceinline__ void store_f8(float* p, const float (&f)[8]) {
  *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(f[4], f[5], f[6], f[7]);
}

// ------------------------------------------------------------------------------------------------
// LayerNorm + modulate, forward: one CTA per token row
// ------------------------------------------------------------------------------------------------
template <int MV>
__global__ void __launch_bounds__(kThreads) ln_modulate_fwd_kernel(
    const bf16* __restrict__ x, const float* __restrict__ shift, const float* __restrict__ scale,
    bf16* __restrict__ y, float* __restrict__ mean_out, float* __restrict__ rstd_out, int D, int L, float eps) {
  __shared__ float red[64];
  const long row = blockIdx.x;
  const long frame = row / L;
  const int nvec = D >> 3;
  const bf16x8* xr = reinterpret_cast<const bf16x8*>(x + row * D);
  float v[MV][8];
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < MV; ++i) {
    const int c = threadIdx.x + i * kThreads;
    if (c < nvec) {
      unpack8(xr[c], v[i]);
#pragma unroll
      for (int j = 0; j < 8; ++j) s += v[i][j];
    }
  }
  const float mean = block_sum(s, red) / D;
  float q = 0.f;
#pragma unroll
  for (int i = 0; i < MV; ++i) {
    const int c = threadIdx.x + i * kThreads;
    if (c < nvec) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float d = v[i][j] - mean;
        q += d * d;
      }
    }
  }
  const float rstd = rsqrtf(block_sum(q, red) / D + eps);
  if (threadIdx.x == 0) {
    mean_out[row] = mean;
    rstd_out[row] = rstd;
  }
  bf16x8* yr = reinterpret_cast<bf16x8*>(y + row * D);
  const float* sh = shift + frame * D;
  const float* sc = scale + frame * D;
#pragma unroll
  for (int i = 0; i < MV; ++i) {
    const int c = threadIdx.x + i * kThreads;
    if (c < nvec) {
      float a[8], b[8], o[8];
      load_f8(sh + c * 8, a);
      load_f8(sc + c * 8, b);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = (v[i][j] - mean) * rstd * (1.f + b[j]) + a[j];
      yr[c] = pack8(o);
    }
  }
}

// Same operator for D <= 2048 with four rows per CTA: the loads of all four rows are in flight together and one pair of block
// reductions serves the four rows, so the memory pipe does not idle behind a reduction per 4 KB row.
constexpr int kLnRows = 4;
__device__ __forceinline__ void block_sum_rows(float (&v)[kLnRows], float* red /* [kLnRows * 32] */) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int r = 0; r < kLnRows; ++r) v[r] = warp_sum(v[r]);
  __syncthreads();
  if (lane == 0) {
#pragma unroll
    for (int r = 0; r < kLnRows; ++r) red[r * 32 + warp] = v[r];
  }
  __syncthreads();
  const int nwarps = (blockDim.x + 31) >> 5;
#pragma unroll
  for (int r = 0; r < kLnRows; ++r) v[r] = warp_sum(lane < nwarps ? red[r * 32 + lane] : 0.f);
}

// A CTA takes `rows_per_cta` consecutive rows of ONE frame, four at a time: every thread keeps the shift / (1 + scale) values of
// its 8 columns in registers for all of them (read per row, the two fp32 modulation vectors are 4x the bytes of the bf16 row and
// made the kernel L2-bound).
__global__ void __launch_bounds__(kThreads) ln_modulate_fwd_rows_kernel(
    const bf16* __restrict__ x, const float* __restrict__ shift, const float* __restrict__ scale,
    bf16* __restrict__ y, float* __restrict__ mean_out, float* __restrict__ rstd_out, int D, int L, int rows_per_cta,
    int groups_per_frame, float eps) {
  __shared__ float red[kLnRows * 32];
  const long frame = blockIdx.x / groups_per_frame;
  const int g = blockIdx.x % groups_per_frame;
  const int r_lo = g * rows_per_cta, r_hi = min(r_lo + rows_per_cta, L);
  const int nvec = D >> 3;
  const int c = threadIdx.x;
  const bool on = c < nvec;
  float a[8], b[8];
  if (on) {
    load_f8(shift + frame * D + c * 8, a);
    load_f8(scale + frame * D + c * 8, b);
#pragma unroll
    for (int j = 0; j < 8; ++j) b[j] += 1.f;
  }
  for (int rb = r_lo; rb < r_hi; rb += kLnRows) {
    const long row0 = frame * L + rb;
    const int n_here = min(kLnRows, r_hi - rb);
    float v[kLnRows][8];
    float s[kLnRows];
#pragma unroll
    for (int r = 0; r < kLnRows; ++r) {
      s[r] = 0.f;
      if (on && r < n_here) {
        unpack8(reinterpret_cast<const bf16x8*>(x + (row0 + r) * D)[c], v[r]);
        const float2 t = add2(add2(CB200_P2(v[r], 0), CB200_P2(v[r], 1)), add2(CB200_P2(v[r], 2), CB200_P2(v[r], 3)));
        s[r] = t.x + t.y;
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) v[r][j] = 0.f;
      }
    }
    block_sum_rows(s, red);
    float mean[kLnRows], q[kLnRows];
#pragma unroll
    for (int r = 0; r < kLnRows; ++r) {
      mean[r] = s[r] / D;
      q[r] = 0.f;
      if (on) {
        // v becomes the centred value; two elements per instruction
        const float2 nm = make_float2(-mean[r], -mean[r]);
        float2 acc = make_float2(0.f, 0.f);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 d = add2(CB200_P2(v[r], j), nm);
          acc = fma2(d, d, acc);
          v[r][2 * j] = d.x;
          v[r][2 * j + 1] = d.y;
        }
        q[r] = acc.x + acc.y;
      }
    }
    block_sum_rows(q, red);
#pragma unroll
    for (int r = 0; r < kLnRows; ++r) {
      if (r >= n_here) break;
      const long row = row0 + r;
      const float rstd = rsqrtf(q[r] / D + eps);
      if (threadIdx.x == 0) {
        mean_out[row] = mean[r];
        rstd_out[row] = rstd;
      }
      if (on) {
        float o[8];
        const float2 rs2 = make_float2(rstd, rstd);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 t = fma2(mul2(CB200_P2(v[r], j), rs2), CB200_P2(b, j), CB200_P2(a, j));
          o[2 * j] = t.x;
          o[2 * j + 1] = t.y;
        }
        reinterpret_cast<bf16x8*>(y + row * D)[c] = pack8(o);
      }
    }
  }
}

// backward: one CTA per group of `rows_per_cta` rows of one frame; writes dx and the per-group
// partials of dshift (sum dy) and dscale (sum dy * xhat) to `partials` [groups, 2, D].
template <int MV>
__global__ void __launch_bounds__(kThreads) ln_modulate_bwd_kernel(
    const bf16* __restrict__ dy, const bf16* __restrict__ x, const float* __restrict__ mean_in,
    const float* __restrict__ rstd_in, const float* __restrict__ scale, bf16* __restrict__ dx,
    float* __restrict__ partials, int D, int L, int rows_per_cta, int groups_per_frame) {
  __shared__ float red[64];
  const long frame = blockIdx.x / groups_per_frame;
  const int g = blockIdx.x % groups_per_frame;
  const int r0 = g * rows_per_cta;
  const int r1 = min(r0 + rows_per_cta, L);
  const int nvec = D >> 3;
  float acc_sh[MV][8], acc_sc[MV][8], onep[MV][8];
#pragma unroll
  for (int i = 0; i < MV; ++i) {
    const int c = threadIdx.x + i * kThreads;
#pragma unroll
    for (int j = 0; j < 8; ++j) acc_sh[i][j] = acc_sc[i][j] = 0.f;
    if (c < nvec) {
      load_f8(scale + frame * D + c * 8, onep[i]);
#pragma unroll
      for (int j = 0; j < 8; ++j) onep[i][j] += 1.f;
    }
  }
  // software pipeline: the loads of row r + 1 are in flight while row r is reduced and written
  bf16x8 nd[MV], nx[MV];
  float nmean = 0.f, nrstd = 0.f;
  auto fetch = [&](int r) {
    const long row = frame * L + r;
    nmean = mean_in[row];
    nrstd = rstd_in[row];
#pragma unroll
    for (int i = 0; i < MV; ++i) {
      const int c = threadIdx.x + i * kThreads;
      if (c < nvec) {
        nd[i] = reinterpret_cast<const bf16x8*>(dy + row * D)[c];
        nx[i] = reinterpret_cast<const bf16x8*>(x + row * D)[c];
      }
    }
  };
  if (r0 < r1) fetch(r0);
  for (int r = r0; r < r1; ++r) {
    const long row = frame * L + r;
    const float mean = nmean, rstd = nrstd;
    bf16x8 cd[MV], cx[MV];
#pragma unroll
    for (int i = 0; i < MV; ++i) {
      cd[i] = nd[i];
      cx[i] = nx[i];
    }
    if (r + 1 < r1) fetch(r + 1);
    float gval[MV][8], xh[MV][8];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < MV; ++i) {
      const int c = threadIdx.x + i * kThreads;
      if (c < nvec) {
        float d[8], xv[8];
        unpack8(cd[i], d);
        unpack8(cx[i], xv);
        const float2 nm = make_float2(-mean, -mean), rs2 = make_float2(rstd, rstd);
        float2 t1 = make_float2(0.f, 0.f), t2 = make_float2(0.f, 0.f);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 dj = CB200_P2(d, j);
          const float2 h = mul2(add2(CB200_P2(xv, j), nm), rs2);
          const float2 sh = add2(CB200_P2(acc_sh[i], j), dj);
          const float2 sc = fma2(dj, h, CB200_P2(acc_sc[i], j));
          const float2 gj = mul2(dj, CB200_P2(onep[i], j));
          t1 = add2(t1, gj);
          t2 = fma2(gj, h, t2);
          xh[i][2 * j] = h.x; xh[i][2 * j + 1] = h.y;
          acc_sh[i][2 * j] = sh.x; acc_sh[i][2 * j + 1] = sh.y;
          acc_sc[i][2 * j] = sc.x; acc_sc[i][2 * j + 1] = sc.y;
          gval[i][2 * j] = gj.x; gval[i][2 * j + 1] = gj.y;
        }
        s1 += t1.x + t1.y;
        s2 += t2.x + t2.y;
      }
    }
    const float2 t = block_sum2(s1, s2, red);
    const float m1 = t.x / D, m2 = t.y / D;
    bf16x8* dxr = reinterpret_cast<bf16x8*>(dx + row * D);
#pragma unroll
    for (int i = 0; i < MV; ++i) {
      const int c = threadIdx.x + i * kThreads;
      if (c < nvec) {
        float o[8];
        const float2 nm1 = make_float2(-m1, -m1), nm2 = make_float2(-m2, -m2), rs2 = make_float2(rstd, rstd);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 t = mul2(rs2, fma2(CB200_P2(xh[i], j), nm2, add2(CB200_P2(gval[i], j), nm1)));
          o[2 * j] = t.x;
          o[2 * j + 1] = t.y;
        }
        dxr[c] = pack8(o);
      }
    }
  }
  float* p = partials + (long)blockIdx.x * 2 * D;
#pragma unroll
  for (int i = 0; i < MV; ++i) {
    const int c = threadIdx.x + i * kThreads;
    if (c < nvec) {
      store_f8(p + c * 8, acc_sh[i]);
      store_f8(p + D + c * 8, acc_sc[i]);
    }
  }
}

// out[frame, k, d] = sum over groups of partials[frame*G + g, k, d]; K slabs per group
__global__ void reduce_partials_kernel(const float* __restrict__ partials, float* __restrict__ out0,
                                       float* __restrict__ out1, int D, int groups_per_frame, int K) {
  const int d = blockIdx.x * blockDim.x + threadIdx.x;
  const long frame = blockIdx.y;
  if (d >= D) return;
  for (int k = 0; k < K; ++k) {
    float s = 0.f;
    const float* p = partials + (frame * groups_per_frame) * (long)K * D + (long)k * D + d;
    for (int g = 0; g < groups_per_frame; ++g) s += p[(long)g * K * D];
    float* o = (k == 0) ? out0 : out1;
    o[frame * D + d] = s;
  }
}

// out[d] = sum over rows of partials[row, d] for many rows and few columns (the weight gradient of the per-head RMSNorm:
// thousands of CTA partials of 64 / 128 columns). A CTA owns 32 columns; 32 warps stride over the rows with coalesced 128-byte
// loads, then the 32 per-warp sums of a column are added in a fixed order: deterministic.
__global__ void __launch_bounds__(1024) reduce_rows_kernel(const float* __restrict__ partials, float* __restrict__ out, int D, int rows) {
  __shared__ float sm[32][33];
  const int lane = threadIdx.x & 31, part = threadIdx.x >> 5;
  const int d = blockIdx.x * 32 + lane;
  float s = 0.f;
  if (d < D)
    for (int r = part; r < rows; r += 32) s += partials[(long)r * D + d];
  sm[part][lane] = s;
  __syncthreads();
  if (part == 0 && d < D) {
    float t = 0.f;
#pragma unroll
    for (int k = 0; k < 32; ++k) t += sm[k][lane];
    out[d] = t;
  }
}

// ------------------------------------------------------------------------------------------------
// gated residual
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads) gate_residual_fwd_kernel(
    const bf16* __restrict__ x, const float* __restrict__ gate, const bf16* __restrict__ y, bf16* __restrict__ out,
    long nvec_total, int D, int L) {
  const int nvec = D >> 3;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec_total; i += (long)gridDim.x * blockDim.x) {
    const long row = i / nvec;
    const int c = (int)(i - row * nvec);
    const long frame = row / L;
    float a[8], b[8], g[8], o[8];
    unpack8(reinterpret_cast<const bf16x8*>(x)[i], a);
    unpack8(reinterpret_cast<const bf16x8*>(y)[i], b);
    load_f8(gate + frame * D + c * 8, g);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = a[j] + g[j] * b[j];
    reinterpret_cast<bf16x8*>(out)[i] = pack8(o);
  }
}

template <int MV>
__global__ void __launch_bounds__(kThreads) gate_residual_bwd_kernel(
    const bf16* __restrict__ dout, const float* __restrict__ gate, const bf16* __restrict__ y, bf16* __restrict__ dy,
    float* __restrict__ partials, int D, int L, int rows_per_cta, int groups_per_frame) {
  const long frame = blockIdx.x / groups_per_frame;
  const int g = blockIdx.x % groups_per_frame;
  const int r0 = g * rows_per_cta, r1 = min(r0 + rows_per_cta, L);
  const int nvec = D >> 3;
  float acc[MV][8], gt[MV][8];
#pragma unroll
  for (int i = 0; i < MV; ++i) {
    const int c = threadIdx.x + i * kThreads;
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;
    if (c < nvec) load_f8(gate + frame * D + c * 8, gt[i]);
  }
  for (int r = r0; r < r1; ++r) {
    const long row = frame * L + r;
    const bf16x8* dor = reinterpret_cast<const bf16x8*>(dout + row * D);
    const bf16x8* yr = reinterpret_cast<const bf16x8*>(y + row * D);
    bf16x8* dyr = reinterpret_cast<bf16x8*>(dy + row * D);
#pragma unroll
    for (int i = 0; i < MV; ++i) {
      const int c = threadIdx.x + i * kThreads;
      if (c < nvec) {
        float d[8], yv[8], o[8];
        unpack8(dor[c], d);
        unpack8(yr[c], yv);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          acc[i][j] += d[j] * yv[j];
          o[j] = d[j] * gt[i][j];
        }
        dyr[c] = pack8(o);
      }
    }
  }
  float* p = partials + (long)blockIdx.x * D;
#pragma unroll
  for (int i = 0; i < MV; ++i) {
    const int c = threadIdx.x + i * kThreads;
    if (c < nvec) store_f8(p + c * 8, acc[i]);
  }
}

// ------------------------------------------------------------------------------------------------
// per-head RMSNorm + RoPE: one warp per (token, head), head_dim in {64, 128}; lane holds HD/32 values
// ------------------------------------------------------------------------------------------------
// Sixteen lanes per (token, head) row, HD / 16 elements (one 16- or 8-byte access) per lane, two rows per warp pass: half the
// instructions per byte of a 32-lane layout (these kernels are bound by instruction issue, not by memory). The rotation partner
// of element i (i +- HD/2) sits in lane ^ 8 at the same register index; reductions stay inside the 16-lane half.
constexpr int kRmsPasses = 4;        // forward: passes (of two rows) whose loads a warp keeps in flight together

template <int E>
__device__ __forceinline__ void load_row_bf16(const bf16* p, float (&v)[E]) {
  if constexpr (E == 8) {
    unpack8(*reinterpret_cast<const bf16x8*>(p), v);
  } else {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
  }
}
template <int E>
__device__ __forceinline__ void store_row_bf16(bf16* p, const float (&o)[E]) {
  if constexpr (E == 8) {
    *reinterpret_cast<bf16x8*>(p) = pack8(o);
  } else {
    uint2 raw;
    *reinterpret_cast<__nv_bfloat162*>(&raw.x) = __floats2bfloat162_rn(o[0], o[1]);
    *reinterpret_cast<__nv_bfloat162*>(&raw.y) = __floats2bfloat162_rn(o[2], o[3]);
    *reinterpret_cast<uint2*>(p) = raw;
  }
}
template <int E>
__device__ __forceinline__ void load_f32_vec(const float* p, float (&v)[E]) {
#pragma unroll
  for (int j = 0; j < E; j += 4) {
    const float4 a = *reinterpret_cast<const float4*>(p + j);
    v[j] = a.x; v[j + 1] = a.y; v[j + 2] = a.z; v[j + 3] = a.w;
  }
}
__device__ __forceinline__ float half_warp_sum(float v) {   // over the 16 lanes of this half
  v += __shfl_xor_sync(0xffffffffu, v, 8);
  v += __shfl_xor_sync(0xffffffffu, v, 4);
  v += __shfl_xor_sync(0xffffffffu, v, 2);
  v += __shfl_xor_sync(0xffffffffu, v, 1);
  return v;
}

template <int HD>
__global__ void __launch_bounds__(256) rmsnorm_rope_fwd_kernel(
    const bf16* __restrict__ x, const float* __restrict__ w, const float* __restrict__ cosv,
    const float* __restrict__ sinv, bf16* __restrict__ y, float* __restrict__ rstd_out, long n_rows, int S, int H,
    float eps) {
  constexpr int E = HD / 16;  // elements per lane (8 or 4)
  constexpr int U = kRmsPasses;
  const int lane = threadIdx.x & 31, sub = lane & 15, half = lane >> 4;
  const long row0 = ((long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * (2 * U) + half;   // this lane's rows: row0 + 2u
  float wv[E];
  load_f32_vec<E>(w + sub * E, wv);
  float v[U][E];
#pragma unroll
  for (int u = 0; u < U; ++u) {
    if (row0 + 2 * u < n_rows) {
      load_row_bf16<E>(x + (row0 + 2 * u) * HD + sub * E, v[u]);
    } else {
#pragma unroll
      for (int j = 0; j < E; ++j) v[u][j] = 0.f;
    }
  }
#pragma unroll
  for (int u = 0; u < U; ++u) {
    const long row = row0 + 2 * u;
    const bool valid = row < n_rows;          // both halves run every shuffle; only the accesses are predicated
    const long s = valid ? (row / H) % S : 0;
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < E; ++j) ss += v[u][j] * v[u][j];
    ss = half_warp_sum(ss);
    const float rstd = rsqrtf(ss / HD + eps);
    if (sub == 0 && valid) rstd_out[row] = rstd;
    float o[E];
#pragma unroll
    for (int j = 0; j < E; ++j) o[j] = v[u][j] * rstd * wv[j];
    if (cosv != nullptr) {
      float c[E], sn[E];
      load_f32_vec<E>(cosv + s * (HD / 2) + (sub & 7) * E, c);
      load_f32_vec<E>(sinv + s * (HD / 2) + (sub & 7) * E, sn);
#pragma unroll
      for (int j = 0; j < E; ++j) {
        const float other = __shfl_xor_sync(0xffffffffu, o[j], 8);
        o[j] = (sub < 8) ? (o[j] * c[j] - other * sn[j]) : (o[j] * c[j] + other * sn[j]);
      }
    }
    if (valid) store_row_bf16<E>(y + row * HD + sub * E, o);
  }
}

// backward: `rows_per_warp` consecutive rows per warp (two per pass) to amortise the weight-gradient partial.
template <int HD>
__global__ void __launch_bounds__(256) rmsnorm_rope_bwd_kernel(
    const bf16* __restrict__ dy, const bf16* __restrict__ x, const float* __restrict__ w,
    const float* __restrict__ rstd_in, const float* __restrict__ cosv, const float* __restrict__ sinv,
    bf16* __restrict__ dx, float* __restrict__ dw_partials, long n_rows, int S, int H, int rows_per_warp) {
  constexpr int E = HD / 16;
  __shared__ float sm[8][HD];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, sub = lane & 15, half = lane >> 4;
  const long warp_global = (long)blockIdx.x * 8 + warp;
  const long r0 = warp_global * rows_per_warp;
  const long r_end = min(r0 + (long)rows_per_warp, n_rows);
  float wv[E], dwacc[E];
  load_f32_vec<E>(w + sub * E, wv);
#pragma unroll
  for (int j = 0; j < E; ++j) dwacc[j] = 0.f;
  constexpr int U = 2;      // passes (of two rows) whose loads are in flight together
  for (long rb = r0; rb < r_end; rb += 2 * U) {
    float dU[U][E], xU[U][E], rsU[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long row = rb + 2 * u + half;
      if (row < r_end) {
        load_row_bf16<E>(dy + row * HD + sub * E, dU[u]);
        load_row_bf16<E>(x + row * HD + sub * E, xU[u]);
        rsU[u] = rstd_in[row];
      } else {
#pragma unroll
        for (int j = 0; j < E; ++j) dU[u][j] = xU[u][j] = 0.f;
        rsU[u] = 0.f;
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long row = rb + 2 * u + half;
      const bool valid = row < r_end;
      const long s = valid ? (row / H) % S : 0;
      float d[E];
#pragma unroll
      for (int j = 0; j < E; ++j) d[j] = dU[u][j];
      if (cosv != nullptr) {
        float c[E], sn[E];
        load_f32_vec<E>(cosv + s * (HD / 2) + (sub & 7) * E, c);
        load_f32_vec<E>(sinv + s * (HD / 2) + (sub & 7) * E, sn);
#pragma unroll
        for (int j = 0; j < E; ++j) {
          const float other = __shfl_xor_sync(0xffffffffu, d[j], 8);
          d[j] = (sub < 8) ? (d[j] * c[j] + other * sn[j]) : (d[j] * c[j] - other * sn[j]);
        }
      }
      const float rstd = rsU[u];
      float dot = 0.f;
      float gv[E];
#pragma unroll
      for (int j = 0; j < E; ++j) {
        dwacc[j] += d[j] * xU[u][j] * rstd;
        gv[j] = d[j] * wv[j];
        dot += gv[j] * xU[u][j];
      }
      dot = half_warp_sum(dot);
      const float k = dot * rstd * rstd * rstd / HD;
      float o[E];
#pragma unroll
      for (int j = 0; j < E; ++j) o[j] = rstd * gv[j] - xU[u][j] * k;
      if (valid) store_row_bf16<E>(dx + row * HD + sub * E, o);
    }
  }
  // the two halves of the warp hold partial sums of the same columns
#pragma unroll
  for (int j = 0; j < E; ++j) dwacc[j] += __shfl_xor_sync(0xffffffffu, dwacc[j], 16);
  if (half == 0) {
#pragma unroll
    for (int j = 0; j < E; ++j) sm[warp][sub * E + j] = dwacc[j];
  }
  __syncthreads();
  if (threadIdx.x < HD) {
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) s += sm[k][threadIdx.x];
    dw_partials[(long)blockIdx.x * HD + threadIdx.x] = s;
  }
}

// ------------------------------------------------------------------------------------------------
// GELU (erf), elementwise
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ float gelu_f(float x) { return 0.5f * x * (1.f + erff(x * 0.70710678118654752f)); }
__device__ __forceinline__ float gelu_grad_f(float x) {
  const float cdf = 0.5f * (1.f + erff(x * 0.70710678118654752f));
  const float pdf = 0.39894228040143268f * __expf(-0.5f * x * x);
  return cdf + x * pdf;
}

__global__ void __launch_bounds__(kThreads) gelu_fwd_kernel(const bf16* __restrict__ x, bf16* __restrict__ y, long nvec) {
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long)gridDim.x * blockDim.x) {
    float a[8];
    unpack8(reinterpret_cast<const bf16x8*>(x)[i], a);
#pragma unroll
    for (int j = 0; j < 8; ++j) a[j] = gelu_f(a[j]);
    reinterpret_cast<bf16x8*>(y)[i] = pack8(a);
  }
}

__global__ void __launch_bounds__(kThreads) gelu_bwd_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x,
                                                             bf16* __restrict__ dx, long nvec) {
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long)gridDim.x * blockDim.x) {
    float a[8], d[8];
    unpack8(reinterpret_cast<const bf16x8*>(x)[i], a);
    unpack8(reinterpret_cast<const bf16x8*>(dy)[i], d);
#pragma unroll
    for (int j = 0; j < 8; ++j) a[j] = d[j] * gelu_grad_f(a[j]);
    reinterpret_cast<bf16x8*>(dx)[i] = pack8(a);
  }
}

__global__ void __launch_bounds__(kThreads) cfg_combine_kernel(const float* __restrict__ c, const float* __restrict__ u,
                                                                float* __restrict__ o, float g, long n) {
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x)
    o[i] = c[i] + g * (c[i] - u[i]);
}

// ------------------------------------------------------------------------------------------------
// optimizer path
// ------------------------------------------------------------------------------------------------
// g32 = scrub(scale * g16); partial[blockIdx] = sum g32^2
__global__ void __launch_bounds__(kThreads) grad_cast_norm_kernel(const bf16* __restrict__ g16, float* __restrict__ g32,
                                                                   float* __restrict__ partials, float scale, long n) {
  __shared__ float red[32];
  float ss = 0.f;
  const long nvec = n >> 3;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long)gridDim.x * blockDim.x) {
    float a[8];
    unpack8(reinterpret_cast<const bf16x8*>(g16)[i], a);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      a[j] = scrub(a[j] * scale);
      ss += a[j] * a[j];
    }
    store_f8(g32 + i * 8, a);
  }
  if (blockIdx.x == 0) {
    for (long i = (nvec << 3) + threadIdx.x; i < n; i += blockDim.x) {
      const float a = scrub(__bfloat162float(g16[i]) * scale);
      g32[i] = a;
      ss += a * a;
    }
  }
  const float t = block_sum(ss, red);
  if (threadIdx.x == 0) partials[blockIdx.x] = t;
}

__global__ void sum_partials_kernel(const float* __restrict__ partials, float* __restrict__ out, int n) {
  __shared__ float red[32];
  float s = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) s += partials[i];
  s = block_sum(s, red);
  if (threadIdx.x == 0) out[0] = s;
}

__global__ void __launch_bounds__(kThreads) adamw_ema_shard_kernel(
    float* __restrict__ master, const float* __restrict__ grad, float* __restrict__ m, float* __restrict__ v,
    float* __restrict__ ema, bf16* __restrict__ out16, const float* __restrict__ clip_coef, float lr, float beta1,
    float beta2, float eps, float wd, float bc1, float rsqrt_bc2, float ema_beta, long n) {
  const float clip = clip_coef ? clip_coef[0] : 1.f;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
    const float g = grad[i] * clip;
    float p = master[i] * (1.f - lr * wd);
    const float mi = beta1 * m[i] + (1.f - beta1) * g;
    const float vi = beta2 * v[i] + (1.f - beta2) * g * g;
    const float denom = sqrtf(vi) * rsqrt_bc2 + eps;
    p -= (lr / bc1) * (mi / denom);
    master[i] = p;
    m[i] = mi;
    v[i] = vi;
    if (ema != nullptr && ema_beta >= 0.f) ema[i] = ema_beta * ema[i] + (1.f - ema_beta) * p;
    if (out16 != nullptr) out16[i] = __float2bfloat16(p);
  }
}

__global__ void __launch_bounds__(kThreads) cast_f32_bf16_kernel(const float* __restrict__ src, bf16* __restrict__ dst, long n) {
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x)
    dst[i] = __float2bfloat16(src[i]);
}

static inline int grid_for(long n, int threads, int max_blocks = 148 * 8) {
  long b = (n + threads - 1) / threads;
  if (b < 1) b = 1;
  return (int)(b > max_blocks ? max_blocks : b);
}

}  // namespace cb200

using namespace cb200;

// ------------------------------------------------------------------------------------------------
// host launchers
// ------------------------------------------------------------------------------------------------
extern "C" {

int cb200_ln_groups_per_frame(int L, int rows_per_cta) { return (L + rows_per_cta - 1) / rows_per_cta; }

void cb200_ln_modulate_fwd(const void* x, const float* shift, const float* scale, void* y, float* mean, float* rstd,
                           long rows, int D, int L, float eps, cudaStream_t st) {
#define LAUNCH(MV) ln_modulate_fwd_kernel<MV><<<(unsigned)rows, kThreads, 0, st>>>((const bf16*)x, shift, scale, (bf16*)y, mean, rstd, D, L, eps)
  if (D <= 2048) {
    constexpr int kRowsPerCta = 32;
    const int G = (L + kRowsPerCta - 1) / kRowsPerCta;
    ln_modulate_fwd_rows_kernel<<<(unsigned)((rows / L) * G), kThreads, 0, st>>>((const bf16*)x, shift, scale, (bf16*)y, mean, rstd, D, L,
                                                                               kRowsPerCta, G, eps);
  } else if (D <= 4096) LAUNCH(2); else LAUNCH(4);
#undef LAUNCH
}

void cb200_ln_modulate_bwd(const void* dy, const void* x, const float* mean, const float* rstd, const float* scale,
                           void* dx, float* dshift, float* dscale, float* partials, long frames, int D, int L,
                           int rows_per_cta, cudaStream_t st) {
  const int G = cb200_ln_groups_per_frame(L, rows_per_cta);
#define LAUNCH(MV) ln_modulate_bwd_kernel<MV><<<(unsigned)(frames * G), kThreads, 0, st>>>((const bf16*)dy, (const bf16*)x, mean, rstd, scale, (bf16*)dx, partials, D, L, rows_per_cta, G)
  if (D <= 2048) LAUNCH(1); else if (D <= 4096) LAUNCH(2); else LAUNCH(4);
#undef LAUNCH
  dim3 grid((D + 255) / 256, (unsigned)frames);
  reduce_partials_kernel<<<grid, 256, 0, st>>>(partials, dshift, dscale, D, G, 2);
}

void cb200_gate_residual_fwd(const void* x, const float* gate, const void* y, void* out, long rows, int D, int L,
                             cudaStream_t st) {
  const long nvec = rows * (D >> 3);
  gate_residual_fwd_kernel<<<grid_for(nvec, kThreads, 148 * 16), kThreads, 0, st>>>((const bf16*)x, gate, (const bf16*)y,
                                                                                    (bf16*)out, nvec, D, L);
}

void cb200_gate_residual_bwd(const void* dout, const float* gate, const void* y, void* dy, float* dgate, float* partials,
                             long frames, int D, int L, int rows_per_cta, cudaStream_t st) {
  const int G = cb200_ln_groups_per_frame(L, rows_per_cta);
#define LAUNCH(MV) gate_residual_bwd_kernel<MV><<<(unsigned)(frames * G), kThreads, 0, st>>>((const bf16*)dout, gate, (const bf16*)y, (bf16*)dy, partials, D, L, rows_per_cta, G)
  if (D <= 2048) LAUNCH(1); else if (D <= 4096) LAUNCH(2); else LAUNCH(4);
#undef LAUNCH
  dim3 grid((D + 255) / 256, (unsigned)frames);
  reduce_partials_kernel<<<grid, 256, 0, st>>>(partials, dgate, nullptr, D, G, 1);
}

void cb200_rmsnorm_rope_fwd(const void* x, const float* w, const float* cosv, const float* sinv, void* y, float* rstd,
                            long n_rows, int S, int H, int HD, float eps, cudaStream_t st) {
  const unsigned blocks = (unsigned)((n_rows + 16 * kRmsPasses - 1) / (16 * kRmsPasses));   // 8 warps x 2 rows x passes per CTA
  if (HD == 128)
    rmsnorm_rope_fwd_kernel<128><<<blocks, 256, 0, st>>>((const bf16*)x, w, cosv, sinv, (bf16*)y, rstd, n_rows, S, H, eps);
  else
    rmsnorm_rope_fwd_kernel<64><<<blocks, 256, 0, st>>>((const bf16*)x, w, cosv, sinv, (bf16*)y, rstd, n_rows, S, H, eps);
}

long cb200_rmsnorm_bwd_blocks(long n_rows, int rows_per_warp) {
  const long warps = (n_rows + rows_per_warp - 1) / rows_per_warp;
  return (warps + 7) / 8;
}

void cb200_rmsnorm_rope_bwd(const void* dy, const void* x, const float* w, const float* rstd, const float* cosv,
                            const float* sinv, void* dx, float* dw, float* partials, long n_rows, int S, int H, int HD,
                            int rows_per_warp, cudaStream_t st) {
  const long blocks = cb200_rmsnorm_bwd_blocks(n_rows, rows_per_warp);
  if (HD == 128)
    rmsnorm_rope_bwd_kernel<128><<<(unsigned)blocks, 256, 0, st>>>((const bf16*)dy, (const bf16*)x, w, rstd, cosv, sinv,
                                                                   (bf16*)dx, partials, n_rows, S, H, rows_per_warp);
  else
    rmsnorm_rope_bwd_kernel<64><<<(unsigned)blocks, 256, 0, st>>>((const bf16*)dy, (const bf16*)x, w, rstd, cosv, sinv,
                                                                  (bf16*)dx, partials, n_rows, S, H, rows_per_warp);
  reduce_rows_kernel<<<(HD + 31) / 32, 1024, 0, st>>>(partials, dw, HD, (int)blocks);
}

void cb200_gelu_fwd(const void* x, void* y, long n, cudaStream_t st) {
  gelu_fwd_kernel<<<grid_for(n >> 3, kThreads, 148 * 16), kThreads, 0, st>>>((const bf16*)x, (bf16*)y, n >> 3);
}

void cb200_gelu_bwd(const void* dy, const void* x, void* dx, long n, cudaStream_t st) {
  gelu_bwd_kernel<<<grid_for(n >> 3, kThreads, 148 * 16), kThreads, 0, st>>>((const bf16*)dy, (const bf16*)x, (bf16*)dx, n >> 3);
}

void cb200_cfg_combine(const float* c, const float* u, float* o, float g, long n, cudaStream_t st) {
  cfg_combine_kernel<<<grid_for(n, kThreads), kThreads, 0, st>>>(c, u, o, g, n);
}

int cb200_grad_cast_norm_blocks(long n) { return grid_for(n >> 3, kThreads, 148 * 4); }

void cb200_grad_cast_norm(const void* g16, float* g32, float* sumsq, float* partials, float scale, long n, cudaStream_t st) {
  const int blocks = cb200_grad_cast_norm_blocks(n);
  grad_cast_norm_kernel<<<blocks, kThreads, 0, st>>>((const bf16*)g16, g32, partials, scale, n);
  sum_partials_kernel<<<1, 256, 0, st>>>(partials, sumsq, blocks);
}

void cb200_adamw_ema_shard(float* master, const float* grad, float* m, float* v, float* ema, void* out16,
                           const float* clip_coef, float lr, float beta1, float beta2, float eps, float wd, long step,
                           float ema_beta, long n, cudaStream_t st) {
  const float bc1 = 1.f - powf(beta1, (float)step);
  const float bc2 = 1.f - powf(beta2, (float)step);
  adamw_ema_shard_kernel<<<grid_for(n, kThreads, 148 * 8), kThreads, 0, st>>>(
      master, grad, m, v, ema, (bf16*)out16, clip_coef, lr, beta1, beta2, eps, wd, bc1, 1.f / sqrtf(bc2), ema_beta, n);
}

void cb200_cast_f32_bf16(const float* src, void* dst, long n, cudaStream_t st) {
  cast_f32_bf16_kernel<<<grid_for(n, kThreads, 148 * 8), kThreads, 0, st>>>(src, (bf16*)dst, n);
}

}  // extern "C"
