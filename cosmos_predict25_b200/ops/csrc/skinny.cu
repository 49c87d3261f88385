// Batched fp32 GEMM for "skinny" problems: a handful of rows (batch x frames of timestep embeddings) against many small weight
// matrices, e.g. the 3 AdaLN-LoRA modulation MLPs of every transformer block and the timestep embedder
// (cosmos_predict2/_src/predict2/networks/minimal_v4_dit.py:776-783, 1131-1162). These run in fp32 (the fp32 island of the
// reference) on a few dozen rows: too few rows for a 128-row tensor-core tile and too many launches as single library GEMMs
// (2 per MLP, 85 MLPs per forward). One launch computes all Z problems
//
//     C[z][r, n] = sum_k fa(A[z][r, k]) * fb(B[z][n, k])  (+ add[r, n] for n < add_cols)
//
// with arbitrary element strides for A and B, so that the same kernel serves the forward (B = weight, k contiguous), the input
// gradient (B = weight read along its rows) and the weight gradient (the reduction runs over the few rows). A is fp32, B is
// bf16 or fp32 and is addressed through a pointer table (weights of different modules) or a base pointer + stride; fa / fb are
// identity or SiLU. Accumulation is fp32 on the CUDA cores in a fixed order: the result is deterministic.

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "launchers.h"

namespace cb200 {

struct SkinnyParams {
  const float* a;
  long a_z, a_r, a_k;
  const long long* b_ptrs;   // per-problem base addresses of B, or nullptr
  const void* b_base;
  long b_z, b_n, b_k;
  void* c;
  long c_z;
  int ldc;
  const float* add;
  int ld_add, add_cols;
  int R, N, K;
  int silu_a, silu_b;
  int ksplit;   // the reduction is cut into this many ranges; range s of problem z writes C[z * ksplit + s]
};

constexpr int kSkTile = 64;     // rows and columns of C per CTA
constexpr int kSkK = 32;        // reduction elements per shared-memory stage
constexpr int kSkLd = kSkTile + 4;

__device__ __forceinline__ float silu_f(float v) { return v / (1.f + __expf(-v)); }
__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ void store_c(float* p, float v) { *p = v; }
__device__ __forceinline__ void store_c(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

template <typename TB, typename TC>
__global__ void __launch_bounds__(256, 2) skinny_bgemm_kernel(SkinnyParams p) {
  __shared__ __align__(16) float As[kSkK][kSkLd];
  __shared__ __align__(16) float Bs[kSkK][kSkLd];
  const int z = blockIdx.z / p.ksplit, ks = blockIdx.z % p.ksplit;
  const int k_per = ((p.K + p.ksplit - 1) / p.ksplit + kSkK - 1) / kSkK * kSkK;
  const int k_lo = ks * k_per, k_hi = min(p.K, k_lo + k_per);
  const int r0 = blockIdx.y * kSkTile, n0 = blockIdx.x * kSkTile;
  const float* A = p.a + (long)z * p.a_z;
  const TB* B = p.b_ptrs ? reinterpret_cast<const TB*>(p.b_ptrs[z]) : reinterpret_cast<const TB*>(p.b_base) + (long)z * p.b_z;
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  // the thread index runs along whichever of (row, k) is contiguous in memory
  const bool a_k_fast = p.a_k == 1, b_k_fast = p.b_k == 1;
  for (int k0 = k_lo; k0 < k_hi; k0 += kSkK) {
#pragma unroll
    for (int it = 0; it < kSkTile * kSkK / 256; ++it) {
      const int idx = it * 256 + tid;
      {
        const int kk = a_k_fast ? idx % kSkK : idx / kSkTile, rr = a_k_fast ? idx / kSkK : idx % kSkTile;
        const int r = r0 + rr, k = k0 + kk;
        float v = 0.f;
        if (r < p.R && k < k_hi) {
          v = A[(long)r * p.a_r + (long)k * p.a_k];
          if (p.silu_a) v = silu_f(v);
        }
        As[kk][rr] = v;
      }
      {
        const int kk = b_k_fast ? idx % kSkK : idx / kSkTile, nn = b_k_fast ? idx / kSkK : idx % kSkTile;
        const int n = n0 + nn, k = k0 + kk;
        float v = 0.f;
        if (n < p.N && k < k_hi) {
          v = to_f32(B[(long)n * p.b_n + (long)k * p.b_k]);
          if (p.silu_b) v = silu_f(v);
        }
        Bs[kk][nn] = v;
      }
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < kSkK; ++kk) {
      const float4 a4 = *reinterpret_cast<const float4*>(&As[kk][ty * 4]);
      const float4 b4 = *reinterpret_cast<const float4*>(&Bs[kk][tx * 4]);
      const float av[4] = {a4.x, a4.y, a4.z, a4.w}, bv[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }
  TC* C = reinterpret_cast<TC*>(p.c) + (long)blockIdx.z * p.c_z;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = r0 + ty * 4 + i;
    if (r >= p.R) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= p.N) continue;
      float v = acc[i][j];
      if (p.add != nullptr && ks == 0 && n < p.add_cols) v += p.add[(long)r * p.ld_add + n];
      store_c(C + (long)r * p.ldc + n, v);
    }
  }
}

}  // namespace cb200

using namespace cb200;

extern "C" int cb200_skinny_bgemm(const float* a, long a_z, long a_r, long a_k, const long long* b_ptrs, const void* b_base, long b_z,
                                  long b_n, long b_k, int b_is_bf16, void* c, long c_z, int ldc, int c_is_bf16, const float* add,
                                  int ld_add, int add_cols, int Z, int R, int N, int K, int silu_a, int silu_b, int ksplit, cudaStream_t st) {
  if (Z <= 0 || R <= 0 || N <= 0 || K <= 0) return 0;
  if (ksplit < 1 || (long)Z * ksplit > 65535 || (R + kSkTile - 1) / kSkTile > 65535) return -1;
  SkinnyParams p{a, a_z, a_r, a_k, b_ptrs, b_base, b_z, b_n, b_k, c, c_z, ldc, add, ld_add, add_cols, R, N, K, silu_a, silu_b, ksplit};
  dim3 grid((N + kSkTile - 1) / kSkTile, (R + kSkTile - 1) / kSkTile, Z * ksplit);
  if (b_is_bf16) {
    if (c_is_bf16) skinny_bgemm_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, 256, 0, st>>>(p);
    else skinny_bgemm_kernel<__nv_bfloat16, float><<<grid, 256, 0, st>>>(p);
  } else {
    if (c_is_bf16) skinny_bgemm_kernel<float, __nv_bfloat16><<<grid, 256, 0, st>>>(p);
    else skinny_bgemm_kernel<float, float><<<grid, 256, 0, st>>>(p);
  }
  return 0;
}
