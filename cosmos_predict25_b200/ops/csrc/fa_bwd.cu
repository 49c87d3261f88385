// Flash attention backward on tcgen05 / TMEM (sm_100a), head_dim 128, bf16, non-causal.
//
// Two deterministic kernels (no atomics, no cross-CTA reduction), each a two-buffer ping-pong between
// one MMA-issuing thread and two 128-thread element-wise groups, like the forward kernel:
//
//   fa_bwd_dq   : a CTA keeps two 128-row query tiles (Q, dO, row statistics) and streams K/V in tiles of 64
//                 keys:  S = Q K^T, dP = dO V^T  ->  dS = P o (dP - delta)  ->  dQ += dS K
//   fa_bwd_dkv  : a CTA keeps one 128-key tile (K, V) and streams Q/dO in tiles of 64 queries; it works on
//                 the transposed problem so that a TMEM lane is a key row:
//                 S^T = K Q^T, dP^T = V dO^T  ->  P^T, dS^T  ->  dV += P^T dO, dK += dS^T Q
//
// P = exp2(S*scale*log2e - lse*log2e) is recomputed from the forward's log-sum-exp; delta = rowsum(dO o O)
// comes from a small preprocessing kernel. bf16 operands P / dS / P^T / dS^T are written by the
// element-wise threads straight into TMEM (over the fp32 scores they were computed from) and consumed by
// tcgen05.mma in its TS form; the N-major B operands (K, Q, dO as [row][d]) are read through MN-major
// shared-memory descriptors of the same TMA tiles that serve as K-major operands elsewhere.
// Recomputing S and dP in both kernels costs 7 GEMMs instead of 5 but removes every dQ atomic.
//
// All waits are bounded and report through `err`.

#include <math.h>

#include "common.cuh"
#include "launchers.h"
#include "sm100.cuh"
#include "tmap.h"

namespace cb200 {
using namespace sm100;

constexpr int kFaBwdDefaultLong = 3;   // kernel used for long key sequences when the caller does not choose

namespace fab {
constexpr int HD = 128;
constexpr int kBig = 128 * HD * 2;    // 32 KB: 128-row tile
constexpr int kSmall = 64 * HD * 2;   // 16 KB: 64-row tile
constexpr int kThreads = 320;
constexpr int kMmaWarp = 9, kTmaWarp = 8;
constexpr int kRingDq = 6;
constexpr int kRingDkv = 8;
constexpr size_t kSmemDq = 4 * (size_t)kBig + kRingDq * (size_t)kSmall + 1024 + 256;
constexpr size_t kSmemDkv = 2 * (size_t)kBig + kRingDkv * (size_t)kSmall + 1024 + 256;
}  // namespace fab

__device__ __forceinline__ float ex2b(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// ------------------------------------------------------------------------------------------------
// preprocessing: delta[b,h,s] = sum_d dO*O ; lse2 = lse * log2(e); both padded to a multiple of 64 rows
// (padding: lse2 = +inf so that recomputed probabilities of out-of-range queries are exactly 0); `sign` = -1 stores both
// negated, which lets the single-pass kernel use packed fused multiply-adds without negations
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) fa_bwd_prep_kernel(const bf16* __restrict__ o, const bf16* __restrict__ d_o,
                                                           const float* __restrict__ lse, float* __restrict__ delta,
                                                           float* __restrict__ lse2, int B, int S, int H, int S_pad, float sign) {
  const int lane = threadIdx.x & 31;
  const long row = (long)blockIdx.x * 8 + (threadIdx.x >> 5);  // over B * H * S_pad
  if (row >= (long)B * H * S_pad) return;
  const int s = (int)(row % S_pad);
  const long bh = row / S_pad;
  const int h = (int)(bh % H);
  const long b = bh / H;
  if (s >= S) {
    if (lane == 0) {
      delta[row] = 0.f;
      lse2[row] = sign * INFINITY;
    }
    return;
  }
  const size_t off = (((size_t)b * S + s) * H + h) * 128 + lane * 4;
  const uint2 ro = *reinterpret_cast<const uint2*>(o + off);
  const uint2 rd = *reinterpret_cast<const uint2*>(d_o + off);
  const float2 o0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&ro.x));
  const float2 o1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&ro.y));
  const float2 d0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&rd.x));
  const float2 d1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&rd.y));
  float acc = o0.x * d0.x + o0.y * d0.y + o1.x * d1.x + o1.y * d1.y;
  acc = warp_sum(acc);
  if (lane == 0) {
    delta[row] = sign * acc;
    lse2[row] = sign * lse[bh * S + s] * 1.4426950408889634f;
  }
}

// ------------------------------------------------------------------------------------------------
// dQ kernel
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(fab::kThreads, 1)
fa_bwd_dq_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_do,
                 const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                 const float* __restrict__ lse2, const float* __restrict__ delta, bf16* __restrict__ dQ, int Sq, int Skv, int H,
                 int Sq_pad, float scale, int* __restrict__ err) {
  using namespace fab;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = smem;                 // 2 x 32 KB
  uint8_t* sdO = smem + 2 * kBig;     // 2 x 32 KB
  uint8_t* sR = smem + 4 * kBig;      // ring: K_0 V_0 K_1 V_1 ... (16 KB each)
  uint64_t* bars = reinterpret_cast<uint64_t*>(sR + kRingDq * kSmall);
  uint64_t* q_full = bars;
  uint64_t* r_full = bars + 1;
  uint64_t* r_empty = r_full + kRingDq;
  uint64_t* s_full = r_empty + kRingDq;   // [2]
  uint64_t* ds_ready = s_full + 2;        // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(ds_ready + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.y, b = blockIdx.z;
  const int q_base = blockIdx.x * 256;
  const int n_kv = (Skv + 63) / 64;
  const float scale_log2 = scale * 1.4426950408889634f;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < kRingDq; ++i) {
      mbar_init(&r_full[i], 1);
      mbar_init(&r_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&ds_ready[i], 4);
    }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == kMmaWarp) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // TMEM columns: S_t = t*128, dP_t = t*128 + 64, dQ_t = 256 + t*128

  if (warp == kTmaWarp) {
    if (lane == 0) {
      prefetch_tmap(&tm_q);
      prefetch_tmap(&tm_do);
      prefetch_tmap(&tm_k);
      prefetch_tmap(&tm_v);
      mbar_arrive_expect_tx(q_full, 4 * kBig);
      for (int t = 0; t < 2; ++t)
        for (int c = 0; c < 2; ++c) {
          tma_load_4d(sQ + t * kBig + c * (kBig / 2), &tm_q, q_full, c * 64, h, q_base + t * 128, b);
          tma_load_4d(sdO + t * kBig + c * (kBig / 2), &tm_do, q_full, c * 64, h, q_base + t * 128, b);
        }
      bool ok = true;
      int slot = 0;
      uint32_t ph = 0;
      for (int n = 0; n < 2 * n_kv; ++n) {
        if (!mbar_wait(&r_empty[slot], ph ^ 1, abort_flag)) { ok = false; break; }
        mbar_arrive_expect_tx(&r_full[slot], kSmall);
        const CUtensorMap* tm = (n & 1) ? &tm_v : &tm_k;
        for (int c = 0; c < 2; ++c) tma_load_4d(sR + slot * kSmall + c * (kSmall / 2), tm, &r_full[slot], c * 64, h, (n >> 1) * 64, b);
        if (++slot == kRingDq) { slot = 0; ph ^= 1; }
      }
      if (!ok) { atomicCAS(err, 0, 21); *abort_flag = 1; }
    }
  } else if (warp == kMmaWarp) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(128, 64, 0, 0);
      constexpr uint32_t idesc_dq = umma_idesc_bf16(128, 128, 0, 1);
      auto issue_s_dp = [&](int t, int k_slot, int v_slot) {
        const uint32_t qa = smem_u32(sQ + t * kBig), da = smem_u32(sdO + t * kBig);
        const uint32_t ka = smem_u32(sR + k_slot * kSmall), va = smem_u32(sR + v_slot * kSmall);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t offa = (kk >> 2) * (kBig / 2) + (kk & 3) * 32, offb = (kk >> 2) * (kSmall / 2) + (kk & 3) * 32;
          umma_ss(tmem_base + t * 128, umma_desc_sw128(qa + offa, 16, 1024), umma_desc_sw128(ka + offb, 16, 1024), idesc_s,
                  kk > 0 ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t offa = (kk >> 2) * (kBig / 2) + (kk & 3) * 32, offb = (kk >> 2) * (kSmall / 2) + (kk & 3) * 32;
          umma_ss(tmem_base + t * 128 + 64, umma_desc_sw128(da + offa, 16, 1024), umma_desc_sw128(va + offb, 16, 1024), idesc_s,
                  kk > 0 ? 1u : 0u);
        }
      };
      auto issue_dq = [&](int t, int k_slot, bool accumulate) {
        const uint32_t ka = smem_u32(sR + k_slot * kSmall);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          umma_ts(tmem_base + 256 + t * 128, tmem_base + t * 128 + kk * 8, umma_desc_sw128(ka + kk * 2048, kSmall / 2, 1024),
                  idesc_dq, (accumulate || kk > 0) ? 1u : 0u);
      };
      bool ok = mbar_wait(q_full, 0, abort_flag);
      int slot = 0;
      uint32_t ph = 0;
      auto take = [&](int& out_slot) -> bool {
        if (!mbar_wait(&r_full[slot], ph, abort_flag)) return false;
        out_slot = slot;
        if (++slot == kRingDq) { slot = 0; ph ^= 1; }
        return true;
      };
      int k_cur = 0, v_cur = 0;
      if (ok) ok = take(k_cur) && take(v_cur);
      if (ok) {
        tc_fence_after();
        issue_s_dp(0, k_cur, v_cur);
        umma_commit(&s_full[0]);
        issue_s_dp(1, k_cur, v_cur);
        umma_commit(&s_full[1]);
        umma_commit(&r_empty[v_cur]);
      }
      for (int j = 0; j < n_kv && ok; ++j) {
        const bool has_next = (j + 1) < n_kv;
        int k_next = 0, v_next = 0;
        if (has_next) {
          ok = take(k_next) && take(v_next);
          if (!ok) break;
        }
        for (int t = 0; t < 2; ++t) {
          if (!mbar_wait(&ds_ready[t], j & 1, abort_flag)) { ok = false; break; }
          tc_fence_after();
          issue_dq(t, k_cur, j > 0);
          if (t == 1) umma_commit(&r_empty[k_cur]);
          if (has_next) issue_s_dp(t, k_next, v_next);
          if (t == 1 && has_next) umma_commit(&r_empty[v_next]);
          umma_commit(&s_full[t]);
        }
        k_cur = k_next;
        v_cur = v_next;
      }
      if (!ok) { atomicCAS(err, 0, 22); *abort_flag = 1; }
    }
  } else {
    const int t = warp >> 2, quarter = warp & 3;
    const int q_row = q_base + t * 128 + quarter * 32 + lane;
    const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
    const uint32_t tS = tmem_base + t * 128 + lane_off;
    const uint32_t tDP = tS + 64;
    const uint32_t tDQ = tmem_base + 256 + t * 128 + lane_off;
    const size_t stat = ((size_t)b * H + h) * Sq_pad + min(q_row, Sq_pad - 1);
    const float my_lse2 = (q_row < Sq_pad) ? lse2[stat] : INFINITY;
    const float my_delta = (q_row < Sq_pad) ? delta[stat] : 0.f;
    bool ok = true;
    for (int j = 0; j < n_kv; ++j) {
      if (!mbar_wait(&s_full[t], j & 1, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const int n_valid = Skv - j * 64;
      uint32_t pk[2][16];
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t s[32], dp[32];
        tmem_ld32(tS + c * 32, s);
        tmem_ld32(tDP + c * 32, dp);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float p0 = ex2b(fmaf(__uint_as_float(s[2 * i]), scale_log2, -my_lse2));
          float p1 = ex2b(fmaf(__uint_as_float(s[2 * i + 1]), scale_log2, -my_lse2));
          if (c * 32 + 2 * i >= n_valid) p0 = 0.f;
          if (c * 32 + 2 * i + 1 >= n_valid) p1 = 0.f;
          const float d0 = p0 * (__uint_as_float(dp[2 * i]) - my_delta);
          const float d1 = p1 * (__uint_as_float(dp[2 * i + 1]) - my_delta);
          __nv_bfloat162 pb = __floats2bfloat162_rn(d0, d1);
          pk[c][i] = *reinterpret_cast<uint32_t*>(&pb);
        }
      }
      // dS overwrites score columns [0,32): only after both score chunks have been read
      tmem_st16(tS, pk[0]);
      tmem_st16(tS + 16, pk[1]);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ds_ready[t]);
    }
    if (ok) ok = mbar_wait(&s_full[t], n_kv & 1, abort_flag);
    if (ok) {
      tc_fence_after();
      bf16* orow = dQ + (((size_t)b * Sq + q_row) * H + h) * HD;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t o[32];
        tmem_ld32(tDQ + c * 32, o);
        tmem_ld_wait();
        if (q_row < Sq) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 ov;
            __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
            for (int i = 0; i < 4; ++i)
              o2[i] = __floats2bfloat162_rn(__uint_as_float(o[q * 8 + 2 * i]) * scale, __uint_as_float(o[q * 8 + 2 * i + 1]) * scale);
            *reinterpret_cast<uint4*>(orow + c * 32 + q * 8) = ov;
          }
        }
      }
    } else if (lane == 0) {
      atomicCAS(err, 0, 23);
      *abort_flag = 1;
    }
  }

  __syncwarp();
  if (*abort_flag) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ------------------------------------------------------------------------------------------------
// dK / dV kernel
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(fab::kThreads, 1)
fa_bwd_dkv_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_do,
                  const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                  const float* __restrict__ lse2, const float* __restrict__ delta, bf16* __restrict__ dK, bf16* __restrict__ dV,
                  int Sq, int Skv, int H, int Sq_pad, float scale, int* __restrict__ err) {
  using namespace fab;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sK = smem;
  uint8_t* sV = smem + kBig;
  uint8_t* sR = smem + 2 * kBig;      // ring: Q_0 dO_0 Q_1 dO_1 ... (16 KB each)
  uint64_t* bars = reinterpret_cast<uint64_t*>(sR + kRingDkv * kSmall);
  uint64_t* kv_full = bars;
  uint64_t* r_full = bars + 1;
  uint64_t* r_empty = r_full + kRingDkv;
  uint64_t* s_full = r_empty + kRingDkv;  // [2]
  uint64_t* p_ready = s_full + 2;         // [2]
  uint64_t* done = p_ready + 2;           // [1]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(done + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.y, b = blockIdx.z;
  const int kv_base = blockIdx.x * 128;
  const int n_q = (Sq + 63) / 64;
  const float scale_log2 = scale * 1.4426950408889634f;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int i = 0; i < kRingDkv; ++i) {
      mbar_init(&r_full[i], 1);
      mbar_init(&r_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&p_ready[i], 4);
    }
    mbar_init(done, 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == kMmaWarp) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // TMEM columns: ST_u = u*128, dPT_u = u*128 + 64, dV = 256, dK = 384

  if (warp == kTmaWarp) {
    if (lane == 0) {
      prefetch_tmap(&tm_q);
      prefetch_tmap(&tm_do);
      prefetch_tmap(&tm_k);
      prefetch_tmap(&tm_v);
      mbar_arrive_expect_tx(kv_full, 2 * kBig);
      for (int c = 0; c < 2; ++c) {
        tma_load_4d(sK + c * (kBig / 2), &tm_k, kv_full, c * 64, h, kv_base, b);
        tma_load_4d(sV + c * (kBig / 2), &tm_v, kv_full, c * 64, h, kv_base, b);
      }
      bool ok = true;
      int slot = 0;
      uint32_t ph = 0;
      for (int n = 0; n < 2 * n_q; ++n) {  // even: Q_i, odd: dO_i
        if (!mbar_wait(&r_empty[slot], ph ^ 1, abort_flag)) { ok = false; break; }
        mbar_arrive_expect_tx(&r_full[slot], kSmall);
        const CUtensorMap* tm = (n & 1) ? &tm_do : &tm_q;
        for (int c = 0; c < 2; ++c) tma_load_4d(sR + slot * kSmall + c * (kSmall / 2), tm, &r_full[slot], c * 64, h, (n >> 1) * 64, b);
        if (++slot == kRingDkv) { slot = 0; ph ^= 1; }
      }
      if (!ok) { atomicCAS(err, 0, 31); *abort_flag = 1; }
    }
  } else if (warp == kMmaWarp) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(128, 64, 0, 0);
      constexpr uint32_t idesc_acc = umma_idesc_bf16(128, 128, 0, 1);
      auto issue_st_dpt = [&](int u, int q_slot, int do_slot) {
        const uint32_t ka = smem_u32(sK), va = smem_u32(sV);
        const uint32_t qa = smem_u32(sR + q_slot * kSmall), da = smem_u32(sR + do_slot * kSmall);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t offa = (kk >> 2) * (kBig / 2) + (kk & 3) * 32, offb = (kk >> 2) * (kSmall / 2) + (kk & 3) * 32;
          umma_ss(tmem_base + u * 128, umma_desc_sw128(ka + offa, 16, 1024), umma_desc_sw128(qa + offb, 16, 1024), idesc_s,
                  kk > 0 ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t offa = (kk >> 2) * (kBig / 2) + (kk & 3) * 32, offb = (kk >> 2) * (kSmall / 2) + (kk & 3) * 32;
          umma_ss(tmem_base + u * 128 + 64, umma_desc_sw128(va + offa, 16, 1024), umma_desc_sw128(da + offb, 16, 1024), idesc_s,
                  kk > 0 ? 1u : 0u);
        }
      };
      auto issue_dv_dk = [&](int u, int q_slot, int do_slot, bool accumulate) {
        const uint32_t qa = smem_u32(sR + q_slot * kSmall), da = smem_u32(sR + do_slot * kSmall);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          umma_ts(tmem_base + 256, tmem_base + u * 128 + kk * 8, umma_desc_sw128(da + kk * 2048, kSmall / 2, 1024), idesc_acc,
                  (accumulate || kk > 0) ? 1u : 0u);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          umma_ts(tmem_base + 384, tmem_base + u * 128 + 64 + kk * 8, umma_desc_sw128(qa + kk * 2048, kSmall / 2, 1024), idesc_acc,
                  (accumulate || kk > 0) ? 1u : 0u);
      };
      bool ok = mbar_wait(kv_full, 0, abort_flag);
      int slot = 0;
      uint32_t ph = 0;
      auto take = [&](int& out_slot) -> bool {
        if (!mbar_wait(&r_full[slot], ph, abort_flag)) return false;
        out_slot = slot;
        if (++slot == kRingDkv) { slot = 0; ph ^= 1; }
        return true;
      };
      int qs[2] = {0, 0}, ds[2] = {0, 0};  // ring slots of the sub-tile currently owned by buffer u
      for (int u = 0; u < 2 && u < n_q && ok; ++u) {
        ok = take(qs[u]) && take(ds[u]);
        if (!ok) break;
        tc_fence_after();
        issue_st_dpt(u, qs[u], ds[u]);
        umma_commit(&s_full[u]);
      }
      for (int i = 0; i < n_q && ok; ++i) {
        const int u = i & 1;
        if (!mbar_wait(&p_ready[u], (i >> 1) & 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        issue_dv_dk(u, qs[u], ds[u], i > 0);
        umma_commit(&r_empty[qs[u]]);
        umma_commit(&r_empty[ds[u]]);
        if (i + 2 < n_q) {
          ok = take(qs[u]) && take(ds[u]);
          if (!ok) break;
          tc_fence_after();
          issue_st_dpt(u, qs[u], ds[u]);
          umma_commit(&s_full[u]);
        }
      }
      if (ok) umma_commit(done);
      if (!ok) { atomicCAS(err, 0, 32); *abort_flag = 1; }
    }
  } else {
    const int u = warp >> 2, quarter = warp & 3;
    const int kv_row = kv_base + quarter * 32 + lane;
    const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
    const uint32_t tST = tmem_base + u * 128 + lane_off;
    const uint32_t tDPT = tST + 64;
    const float* lse_bh = lse2 + ((size_t)b * H + h) * Sq_pad;
    const float* del_bh = delta + ((size_t)b * H + h) * Sq_pad;
    bool ok = true;
    for (int i = u; i < n_q; i += 2) {
      if (!mbar_wait(&s_full[u], (i >> 1) & 1, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const float4* l4 = reinterpret_cast<const float4*>(lse_bh + i * 64);
      const float4* d4 = reinterpret_cast<const float4*>(del_bh + i * 64);
      uint32_t pp[2][16], pd[2][16];
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t s[32], dp[32];
        tmem_ld32(tST + c * 32, s);
        tmem_ld32(tDPT + c * 32, dp);
        tmem_ld_wait();
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          const float4 lv = __ldg(l4 + c * 8 + g);
          const float4 dv = __ldg(d4 + c * 8 + g);
          const float ls[4] = {lv.x, lv.y, lv.z, lv.w};
          const float de[4] = {dv.x, dv.y, dv.z, dv.w};
          float p[4], d[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            p[e] = ex2b(fmaf(__uint_as_float(s[g * 4 + e]), scale_log2, -ls[e]));
            d[e] = p[e] * (__uint_as_float(dp[g * 4 + e]) - de[e]);
          }
          __nv_bfloat162 a0 = __floats2bfloat162_rn(p[0], p[1]), a1 = __floats2bfloat162_rn(p[2], p[3]);
          __nv_bfloat162 b0 = __floats2bfloat162_rn(d[0], d[1]), b1 = __floats2bfloat162_rn(d[2], d[3]);
          pp[c][g * 2] = *reinterpret_cast<uint32_t*>(&a0);
          pp[c][g * 2 + 1] = *reinterpret_cast<uint32_t*>(&a1);
          pd[c][g * 2] = *reinterpret_cast<uint32_t*>(&b0);
          pd[c][g * 2 + 1] = *reinterpret_cast<uint32_t*>(&b1);
        }
      }
      // P^T / dS^T overwrite columns [0,32) of the fp32 tiles: only after both chunks have been read
      tmem_st16(tST, pp[0]);
      tmem_st16(tST + 16, pp[1]);
      tmem_st16(tDPT, pd[0]);
      tmem_st16(tDPT + 16, pd[1]);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_ready[u]);
    }
    if (ok) ok = mbar_wait(done, 0, abort_flag);
    if (ok) {
      tc_fence_after();
      // warps 0-3 write dV, warps 4-7 write dK (scaled)
      const uint32_t tAcc = tmem_base + 256 + u * 128 + lane_off;
      const float mul = (u == 0) ? 1.f : scale;
      bf16* base = (u == 0) ? dV : dK;
      bf16* orow = base + (((size_t)b * Skv + kv_row) * H + h) * HD;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t o[32];
        tmem_ld32(tAcc + c * 32, o);
        tmem_ld_wait();
        if (kv_row < Skv) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 ov;
            __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
            for (int e = 0; e < 4; ++e)
              o2[e] = __floats2bfloat162_rn(__uint_as_float(o[q * 8 + 2 * e]) * mul, __uint_as_float(o[q * 8 + 2 * e + 1]) * mul);
            *reinterpret_cast<uint4*>(orow + c * 32 + q * 8) = ov;
          }
        }
      }
    } else if (lane == 0) {
      atomicCAS(err, 0, 33);
      *abort_flag = 1;
    }
  }

  __syncwarp();
  if (*abort_flag) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace cb200

using namespace cb200;

extern "C" int cb200_fa_bwd_fused_main(const void* d_o, const void* q, const void* k, const void* v, const float* lse2,
                                       const float* delta, float* dq_acc, void* dq, void* dk, void* dv, int B, int Sq, int Skv, int H,
                                       int S_pad, float scale, int dbg, int* err, cudaStream_t st);

extern "C" int cb200_fa_bwd_tile_main(const void* d_o, const void* q, const void* k, const void* v, const float* lse2,
                                      const float* delta, float* dq_acc, void* dk, void* dv, int B, int Sq, int Skv, int H, int S_pad,
                                      float scale, int* err, cudaStream_t st);
extern "C" void cb200_fa_bwd_dq_convert(const float* acc, void* dq, int B, int S, int H, float scale, cudaStream_t st);

// variant 0: choose by problem size; 1: two deterministic kernels (7 GEMMs, no atomics); 2: single pass over 128 x 64 sub-tiles with
// fp32 dQ accumulation (5 GEMMs); 3: single pass over 128 x 128 tiles (5 GEMMs, every MMA N = 128)
static int fa_bwd_pick(int Skv, int variant) { return variant != 0 ? variant : (Skv >= 2048 ? kFaBwdDefaultLong : 1); }
static bool fa_bwd_use_fused(int Skv, int variant) { return fa_bwd_pick(Skv, variant) >= 2; }

extern "C" long cb200_fa_bwd_scratch_floats_v(int B, int Sq, int Skv, int H, int variant) {
  const long S_pad = (Sq + 127) / 128 * 128;
  long n = 2L * B * H * S_pad;
  if (fa_bwd_use_fused(Skv, variant)) n += (long)B * Sq * H * 128;
  return n;
}

extern "C" int cb200_fa_bwd_scratch_floats(int B, int Sq, int H) {
  const int S_pad = (Sq + 127) / 128 * 128;
  return 2 * B * H * S_pad;
}

// q, o, do, dq [B,Sq,H,128]; k, v, dk, dv [B,Skv,H,128]; lse [B,H,Sq]; scratch: cb200_fa_bwd_scratch_floats floats
extern "C" int cb200_fa_bwd_v(const void* d_o, const void* q, const void* k, const void* v, const void* o, const float* lse, void* dq,
                              void* dk, void* dv, float* scratch, int B, int Sq, int Skv, int H, float scale, int variant, int* err,
                              cudaStream_t st);

extern "C" int cb200_fa_bwd(const void* d_o, const void* q, const void* k, const void* v, const void* o, const float* lse, void* dq,
                            void* dk, void* dv, float* scratch, int B, int Sq, int Skv, int H, float scale, int* err,
                            cudaStream_t st) {
  return cb200_fa_bwd_v(d_o, q, k, v, o, lse, dq, dk, dv, scratch, B, Sq, Skv, H, scale, 1, err, st);
}

// scratch: cb200_fa_bwd_scratch_floats_v(B, Sq, Skv, H, variant) floats
extern "C" int cb200_fa_bwd_v(const void* d_o, const void* q, const void* k, const void* v, const void* o, const float* lse, void* dq,
                              void* dk, void* dv, float* scratch, int B, int Sq, int Skv, int H, float scale, int variant, int* err,
                              cudaStream_t st) {
  using namespace fab;
  const int S_pad = (Sq + 127) / 128 * 128;
  float* delta = scratch;
  float* lse2 = scratch + (size_t)B * H * S_pad;
  {
    const long rows = (long)B * H * S_pad;
    fa_bwd_prep_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, st>>>((const bf16*)o, (const bf16*)d_o, lse, delta, lse2, B, Sq, H, S_pad,
                                                                   fa_bwd_use_fused(Skv, variant) ? -1.f : 1.f);
  }
  if (fa_bwd_pick(Skv, variant) == 3) {
    float* acc = scratch + 2 * (size_t)B * H * S_pad;
    const int rc = cb200_fa_bwd_tile_main(d_o, q, k, v, lse2, delta, acc, dk, dv, B, Sq, Skv, H, S_pad, scale, err, st);
    if (rc) return rc;
    cb200_fa_bwd_dq_convert(acc, dq, B, Sq, H, scale, st);
    return (int)cudaGetLastError();
  }
  if (fa_bwd_use_fused(Skv, variant))
    return cb200_fa_bwd_fused_main(d_o, q, k, v, lse2, delta, scratch + 2 * (size_t)B * H * S_pad, dq, dk, dv, B, Sq, Skv, H, S_pad, scale,
                                   0, err, st);
  auto make = [&](CUtensorMap* m, const void* p, int S, int box_rows) {
    const uint64_t dims[4] = {(uint64_t)HD, (uint64_t)H, (uint64_t)S, (uint64_t)B};
    const uint64_t strides[3] = {(uint64_t)HD * 2, (uint64_t)H * HD * 2, (uint64_t)S * H * HD * 2};
    const uint32_t box[4] = {64, 1, (uint32_t)box_rows, 1};
    return make_tmap_bf16(m, p, 4, dims, strides, box);
  };
  CUtensorMap q128, do128, k64, v64, q64, do64, k128, v128;
  int rc = 0;
  rc |= make(&q128, q, Sq, 128);
  rc |= make(&do128, d_o, Sq, 128);
  rc |= make(&k64, k, Skv, 64);
  rc |= make(&v64, v, Skv, 64);
  rc |= make(&q64, q, Sq, 64);
  rc |= make(&do64, d_o, Sq, 64);
  rc |= make(&k128, k, Skv, 128);
  rc |= make(&v128, v, Skv, 128);
  if (rc) return rc;
  static bool attr = false;
  if (!attr) {
    cudaError_t e = cudaFuncSetAttribute(fa_bwd_dq_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemDq);
    if (e != cudaSuccess) return 100 + (int)e;
    e = cudaFuncSetAttribute(fa_bwd_dkv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemDkv);
    if (e != cudaSuccess) return 200 + (int)e;
    attr = true;
  }
  dim3 grid_q((Sq + 255) / 256, H, B);
  fa_bwd_dq_kernel<<<grid_q, kThreads, kSmemDq, st>>>(q128, do128, k64, v64, lse2, delta, (bf16*)dq, Sq, Skv, H, S_pad, scale, err);
  dim3 grid_kv((Skv + 127) / 128, H, B);
  fa_bwd_dkv_kernel<<<grid_kv, kThreads, kSmemDkv, st>>>(q64, do64, k128, v128, lse2, delta, (bf16*)dk, (bf16*)dv, Sq, Skv, H, S_pad,
                                                         scale, err);
  return (int)cudaGetLastError();
}

// Neighbourhood attention backward on tensors in tile order (see cb200_fa_bwd_tile_na): statistics, tile-sparse single-pass
// kernel, dQ conversion. scratch: 2 * B * H * S + B * S * H * 128 floats.
extern "C" int cb200_fa_bwd_tile_na(const void* d_o, const void* q, const void* k, const void* v, const float* lse2, const float* delta,
                                    float* dq_acc, void* dk, void* dv, int B, int S, int H, float scale, const int* q_list,
                                    const int* q_cnt, int max_n, const uint8_t* bt, const uint8_t* bh, const uint8_t* bw, int nT, int nH,
                                    int nW, int* err, cudaStream_t st);

extern "C" long cb200_fa_bwd_na_scratch_floats(int B, int S, int H) { return 2L * B * H * S + (long)B * S * H * 128; }

extern "C" int cb200_fa_bwd_na(const void* d_o, const void* q, const void* k, const void* v, const void* o, const float* lse, void* dq,
                               void* dk, void* dv, float* scratch, int B, int S, int H, float scale, const int* q_list,
                               const int* q_cnt, int max_n, const uint8_t* bt, const uint8_t* bh, const uint8_t* bw, int nT, int nH,
                               int nW, int* err, cudaStream_t st) {
  if (S % 128 != 0) return -41;
  float* delta = scratch;
  float* lse2 = scratch + (size_t)B * H * S;
  float* acc = scratch + 2 * (size_t)B * H * S;
  const long rows = (long)B * H * S;
  fa_bwd_prep_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, st>>>((const bf16*)o, (const bf16*)d_o, lse, delta, lse2, B, S, H, S, -1.f);
  const int rc = cb200_fa_bwd_tile_na(d_o, q, k, v, lse2, delta, acc, dk, dv, B, S, H, scale, q_list, q_cnt, max_n, bt, bh, bw, nT, nH, nW,
                                      err, st);
  if (rc) return rc;
  cb200_fa_bwd_dq_convert(acc, dq, B, S, H, scale, st);
  return (int)cudaGetLastError();
}
