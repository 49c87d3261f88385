// Flash attention backward in ONE pass over the score matrix (5 GEMMs per tile), tcgen05 / TMEM, sm_100a,
// head_dim 128, bf16, non-causal.
//
// A CTA owns one tile of 128 keys (K, V resident in shared memory, dK and dV accumulated in TMEM) and streams
// the queries in sub-tiles of 64. It works on the transposed problem, so a TMEM lane is a key row:
//
//   S^T = K Q^T, dP^T = V dO^T           (SS MMAs, 128 x 64 x 128)
//   P^T = exp2(S^T*c - lse), dS^T = P^T o (dP^T - delta)      (element-wise warps, one key row per thread)
//   dV += P^T dO, dK += dS^T Q           (TS MMAs: P^T / dS^T are bf16 in TMEM, written over the fp32 scores)
//   dQ^T = K^T dS^T                      (SS MMA: K^T is the resident K tile read M-major, dS^T a 16 KB
//                                         shared-memory tile written by the element-wise warps)
//
// dQ^T of a sub-tile is a [128 d x 64 q] fp32 block in TMEM; the element-wise warps read it back (lane = d) and
// add it into an fp32 dQ buffer in global memory with red.global.add (32 consecutive d per warp instruction =
// one 128-byte line). A small kernel converts that buffer to bf16 at the end.
//
// TMEM (512 columns): buffer u in {0,1} at u*128: S^T fp32 [0,64), dP^T fp32 [64,128); after the element-wise
// pass P^T bf16 sits in [0,32), dS^T bf16 in [32,64) and the freed half [64,128) receives dQ^T, so the next S^T can be
// issued without waiting for the dQ^T read-back (only the next dP^T waits for it);
// dV = [256,384), dK = [384,512). Two buffers ping-pong between the MMA thread and two 8-warp groups (two warps per
// TMEM lane quarter, 32 query columns each: the element-wise pass is latency-bound, so it is spread over 16 warps).
//
// All waits are bounded and report through `err`.

#include <math.h>

#include <algorithm>

#include "common.cuh"
#include "launchers.h"
#include "sm100.cuh"
#include "tmap.h"

namespace cb200 {
using namespace sm100;

namespace faf {
constexpr int HD = 128;
constexpr int kBig = 128 * HD * 2;    // 32 KB
constexpr int kSmall = 64 * HD * 2;   // 16 KB
constexpr int kThreads = 576;          // 16 element-wise warps + TMA warp + MMA warp
constexpr int kMmaWarp = 17, kTmaWarp = 16;
constexpr int kRing = 7;
constexpr int kStat = 512;            // per ring slot: 64 lse2 + 64 delta floats
constexpr size_t kSmem = 2 * (size_t)kBig + kRing * (size_t)kSmall + 2 * (size_t)kSmall + kRing * (size_t)kStat + 1024 + 512;
}  // namespace faf

__device__ __forceinline__ float ex2f(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void red_add_f32(float* p, float v) {
  asm volatile("red.global.add.f32 [%0], %1;" ::"l"(p), "f"(v) : "memory");
}

__global__ void __launch_bounds__(faf::kThreads, 1)
fa_bwd_fused_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_do,
                    const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                    const float* __restrict__ lse2, const float* __restrict__ delta, float* __restrict__ dQacc,
                    bf16* __restrict__ dK, bf16* __restrict__ dV, int Sq, int Skv, int H, int Sq_pad, float scale,
                    int* __restrict__ err) {
  using namespace faf;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sK = smem;
  uint8_t* sV = smem + kBig;
  uint8_t* sR = smem + 2 * kBig;                 // ring: Q_0 dO_0 Q_1 dO_1 ... (16 KB each)
  uint8_t* sDS = sR + kRing * kSmall;            // dS^T tiles [128 keys][64 queries] bf16, one per buffer
  float* sStat = reinterpret_cast<float*>(sDS + 2 * kSmall);
  uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(sStat) + kRing * kStat);
  uint64_t* kv_full = bars;
  uint64_t* r_full = bars + 1;
  uint64_t* r_empty = r_full + kRing;
  uint64_t* s_full = r_empty + kRing;   // [2] S^T / dP^T written
  uint64_t* p_ready = s_full + 2;       // [2] P^T / dS^T written (8 warps)
  uint64_t* dq_full = p_ready + 2;      // [2] dQ^T written
  uint64_t* dq_free = dq_full + 2;      // [2] dQ^T read back (8 warps)
  uint64_t* done = dq_free + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(done + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  // the shuffle makes the warp index (and every role branch below) provably warp-uniform for the compiler
  const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;
  const int h = blockIdx.y, b = blockIdx.z;
  const int kv_base = blockIdx.x * 128;
  const int n_q = (Sq + 63) / 64;
  const float scale_log2 = scale * 1.4426950408889634f;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int i = 0; i < kRing; ++i) {
      mbar_init(&r_full[i], 1);
      mbar_init(&r_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&p_ready[i], 8);
      mbar_init(&dq_full[i], 1);
      mbar_init(&dq_free[i], 8);
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
  const size_t bh = (size_t)b * H + h;

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
      for (int n = 0; n < 2 * n_q; ++n) {  // even: Q_i (+ row statistics), odd: dO_i
        if (!mbar_wait(&r_empty[slot], ph ^ 1, abort_flag)) { ok = false; break; }
        const bool is_q = (n & 1) == 0;
        mbar_arrive_expect_tx(&r_full[slot], kSmall + (is_q ? kStat : 0));
        const CUtensorMap* tm = is_q ? &tm_q : &tm_do;
        for (int c = 0; c < 2; ++c) tma_load_4d(sR + slot * kSmall + c * (kSmall / 2), tm, &r_full[slot], c * 64, h, (n >> 1) * 64, b);
        if (is_q) {
          float* st = sStat + slot * (kStat / 4);
          bulk_load_1d(st, lse2 + bh * Sq_pad + (size_t)(n >> 1) * 64, 256, &r_full[slot]);
          bulk_load_1d(st + 64, delta + bh * Sq_pad + (size_t)(n >> 1) * 64, 256, &r_full[slot]);
        }
        if (++slot == kRing) { slot = 0; ph ^= 1; }
      }
      if (!ok) { atomicCAS(err, 0, 41); *abort_flag = 1; }
    }
  } else if (warp == kMmaWarp) {
    {
      // the whole warp runs this code with identical values; only `leader` issues (see umma_ss_w)
      const uint32_t leader = elect_one() ? 1u : 0u;
      // votes keep the loop conditions warp-uniform
      auto wait_all = [&](uint64_t* bar, uint32_t parity) -> bool { return __all_sync(0xffffffffu, mbar_wait(bar, parity, abort_flag)); };
      constexpr uint32_t idesc_s = umma_idesc_bf16(128, 64, 0, 0);
      constexpr uint32_t idesc_acc = umma_idesc_bf16(128, 128, 0, 1);
      constexpr uint32_t idesc_dq = umma_idesc_bf16(128, 64, 1, 1);
      // Base descriptors are built once; an operand slice is the base plus a constant added to the address field (16-byte
      // units, no carry out of the field because shared memory is smaller than 256 KB).
      const uint64_t dK_km = umma_desc_sw128(smem_u32(sK), 16, 1024);            // K  as K-major A   (S^T)
      const uint64_t dV_km = umma_desc_sw128(smem_u32(sV), 16, 1024);            // V  as K-major A   (dP^T)
      const uint64_t dK_mn = umma_desc_sw128(smem_u32(sK), kBig / 2, 1024);      // K^T as M-major A  (dQ^T)
      const uint64_t dR_km = umma_desc_sw128(smem_u32(sR), 16, 1024);            // ring slot as K-major B  (Q in S^T, dO in dP^T)
      const uint64_t dR_mn = umma_desc_sw128(smem_u32(sR), kSmall / 2, 1024);    // ring slot as N-major B  (dO in dV, Q in dK)
      const uint64_t dDS_mn = umma_desc_sw128(smem_u32(sDS), kSmall / 2, 1024);  // dS^T tile as N-major B  (dQ^T)
      auto issue_st = [&](int u, int q_slot) {
        const uint64_t bq = dR_km + (uint64_t)(q_slot * (kSmall >> 4));
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t offa = ((kk >> 2) * (kBig / 2) + (kk & 3) * 32) >> 4, offb = ((kk >> 2) * (kSmall / 2) + (kk & 3) * 32) >> 4;
          umma_ss_w(tmem_base + u * 128, dK_km + offa, bq + offb, idesc_s, kk > 0 ? 1u : 0u, leader);
        }
      };
      auto issue_dpt = [&](int u, int do_slot) {
        const uint64_t bd = dR_km + (uint64_t)(do_slot * (kSmall >> 4));
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t offa = ((kk >> 2) * (kBig / 2) + (kk & 3) * 32) >> 4, offb = ((kk >> 2) * (kSmall / 2) + (kk & 3) * 32) >> 4;
          umma_ss_w(tmem_base + u * 128 + 64, dV_km + offa, bd + offb, idesc_s, kk > 0 ? 1u : 0u, leader);
        }
      };
      // dQ^T[d, q] = sum_kv K[kv, d] dS^T[kv, q]: A = K tile read M-major (two 64-wide d chunks, 16 keys per step),
      // B = dS^T tile read N-major (one 64-wide q chunk)
      auto issue_dq = [&](int u) {
        const uint64_t bs = dDS_mn + (uint64_t)(u * (kSmall >> 4));
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          umma_ss_w(tmem_base + u * 128 + 64, dK_mn + (uint32_t)(kk * (2048 >> 4)), bs + (uint32_t)(kk * (2048 >> 4)), idesc_dq,
                    kk > 0 ? 1u : 0u, leader);
      };
      auto issue_dv_dk = [&](int u, int q_slot, int do_slot, bool accumulate) {
        const uint64_t bq = dR_mn + (uint64_t)(q_slot * (kSmall >> 4)), bd = dR_mn + (uint64_t)(do_slot * (kSmall >> 4));
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          umma_ts_w(tmem_base + 256, tmem_base + u * 128 + kk * 8, bd + (uint32_t)(kk * (2048 >> 4)), idesc_acc,
                    (accumulate || kk > 0) ? 1u : 0u, leader);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          umma_ts_w(tmem_base + 384, tmem_base + u * 128 + 32 + kk * 8, bq + (uint32_t)(kk * (2048 >> 4)), idesc_acc,
                    (accumulate || kk > 0) ? 1u : 0u, leader);
      };
      bool ok = wait_all(kv_full, 0);
      int slot = 0;
      uint32_t ph = 0;
      auto take = [&](int& out_slot) -> bool {
        if (!wait_all(&r_full[slot], ph)) return false;
        out_slot = slot;
        if (++slot == kRing) { slot = 0; ph ^= 1; }
        return true;
      };
      int qs[2] = {0, 0}, ds[2] = {0, 0};
      for (int u = 0; u < 2 && u < n_q && ok; ++u) {
        ok = take(qs[u]) && take(ds[u]);
        if (!ok) break;
        tc_fence_after();
        issue_st(u, qs[u]);
        issue_dpt(u, ds[u]);
        umma_commit_w(&s_full[u], leader);
      }
      for (int i = 0; i < n_q && ok; ++i) {
        const int u = i & 1;
        const uint32_t par = (i >> 1) & 1;
        if (!wait_all(&p_ready[u], par)) { ok = false; break; }
        tc_fence_after();
        issue_dq(u);
        umma_commit_w(&dq_full[u], leader);
        issue_dv_dk(u, qs[u], ds[u], i > 0);
        umma_commit_w(&r_empty[qs[u]], leader);
        umma_commit_w(&r_empty[ds[u]], leader);
        if (i + 2 < n_q) {
          ok = take(qs[u]) && take(ds[u]);
          if (!ok) break;
          // S^T only overwrites P^T / dS^T, which the MMAs just issued consume in order: no wait. dP^T overwrites the
          // columns that hold dQ^T of this sub-tile, so it waits for the read-back (hidden behind dV / dK / S^T).
          tc_fence_after();
          issue_st(u, qs[u]);
          if (!wait_all(&dq_free[u], par)) { ok = false; break; }
          tc_fence_after();
          issue_dpt(u, ds[u]);
          umma_commit_w(&s_full[u], leader);
        }
      }
      if (ok) umma_commit_w(done, leader);
      if (!ok && lane == 0) { atomicCAS(err, 0, 42); *abort_flag = 1; }
    }
  } else {
    // ------------------------------------------------------------------ element-wise groups
    // 8 warps per buffer: warp pair (half = 0 / 1) shares a lane quarter and splits the 64 query columns, so a thread
    // handles one key row x 32 queries (two chunks of 16).
    const int u = warp >> 3, quarter = warp & 3, half = (warp >> 2) & 1;
    const int row = quarter * 32 + lane;            // key row inside the tile == TMEM lane == d index when draining dQ^T
    const int kv_row = kv_base + row;
    const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
    const uint32_t tST = tmem_base + u * 128 + lane_off;
    const uint32_t tDPT = tST + 64;
    uint8_t* ds_row = sDS + u * kSmall + row * 128;
    const int sw = row & 7;
    const int pair_bar = 1 + u * 4 + quarter;       // named barrier of the two warps that share these TMEM lanes
    bool ok = true;
    for (int i = u; i < n_q; i += 2) {
      const uint32_t par = (i >> 1) & 1;
      const int n = 2 * i;                                  // ring sequence number of Q_i
      const int qslot = n % kRing;
      if (!mbar_wait(&s_full[u], par, abort_flag)) { ok = false; break; }
      if (!mbar_wait(&r_full[qslot], (n / kRing) & 1, abort_flag)) { ok = false; break; }  // row statistics landed
      tc_fence_after();
      const float4* l4 = reinterpret_cast<const float4*>(sStat + qslot * (kStat / 4)) + half * 8;
      const float4* d4 = l4 + 16;
      uint32_t pp[16], pd[16];
      const float2 sc2 = make_float2(scale_log2, scale_log2);
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t s[16], dp[16];
        tmem_ld16(tST + half * 32 + c * 16, s);
        tmem_ld16(tDPT + half * 32 + c * 16, dp);
        tmem_ld_wait();
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          const float4 nl = l4[c * 4 + g];   // -lse * log2(e)
          const float4 nd = d4[c * 4 + g];   // -delta
          // packed f32x2 arithmetic: the element-wise pass is bound by instruction issue
          const float2 x0 = fma2(make_float2(__uint_as_float(s[g * 4]), __uint_as_float(s[g * 4 + 1])), sc2, make_float2(nl.x, nl.y));
          const float2 x1 = fma2(make_float2(__uint_as_float(s[g * 4 + 2]), __uint_as_float(s[g * 4 + 3])), sc2, make_float2(nl.z, nl.w));
          const float2 p0 = make_float2(ex2f(x0.x), ex2f(x0.y)), p1 = make_float2(ex2f(x1.x), ex2f(x1.y));
          const float2 t0 = add2(make_float2(__uint_as_float(dp[g * 4]), __uint_as_float(dp[g * 4 + 1])), make_float2(nd.x, nd.y));
          const float2 t1 = add2(make_float2(__uint_as_float(dp[g * 4 + 2]), __uint_as_float(dp[g * 4 + 3])), make_float2(nd.z, nd.w));
          const float2 d0 = mul2(p0, t0), d1 = mul2(p1, t1);
          __nv_bfloat162 a0 = __floats2bfloat162_rn(p0.x, p0.y), a1 = __floats2bfloat162_rn(p1.x, p1.y);
          __nv_bfloat162 b0 = __floats2bfloat162_rn(d0.x, d0.y), b1 = __floats2bfloat162_rn(d1.x, d1.y);
          pp[c * 8 + g * 2] = *reinterpret_cast<uint32_t*>(&a0);
          pp[c * 8 + g * 2 + 1] = *reinterpret_cast<uint32_t*>(&a1);
          pd[c * 8 + g * 2] = *reinterpret_cast<uint32_t*>(&b0);
          pd[c * 8 + g * 2 + 1] = *reinterpret_cast<uint32_t*>(&b1);
        }
      }
      // P^T -> [0,32) and dS^T -> [32,64) overwrite fp32 scores that the partner warp reads: both must have loaded first
      asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory");
      tmem_st16(tST + half * 16, pp);
      tmem_st16(tST + 32 + half * 16, pd);
#pragma unroll
      for (int j = 0; j < 4; ++j) {  // 16-byte chunk (half*4 + j) = queries half*32 + 8j .. +7, 128-byte swizzle
        const uint4 v = make_uint4(pd[j * 4], pd[j * 4 + 1], pd[j * 4 + 2], pd[j * 4 + 3]);
        *reinterpret_cast<uint4*>(ds_row + (((half * 4 + j) ^ sw) << 4)) = v;
      }
      fence_proxy_async();
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_ready[u]);

      // ---- read this warp's half of dQ^T back (lane = d) and add it into the fp32 dQ buffer
      if (!mbar_wait(&dq_full[u], par, abort_flag)) { ok = false; break; }
      tc_fence_after();
      uint32_t a[32];
      tmem_ld32(tST + 64 + half * 32, a);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&dq_free[u]);
      const int q0 = i * 64 + half * 32;
      // head-major accumulator [B, H, Sq, 128]: consecutive queries are 512 bytes apart, so every reduction below is one
      // instruction with an immediate offset from a single base pointer
      float* qrow = dQacc + (bh * Sq + (size_t)q0) * HD + row;
      const int n_valid = min(32, Sq - q0);
      if (n_valid == 32) {
#pragma unroll
        for (int j = 0; j < 32; ++j) red_add_f32(qrow + j * HD, __uint_as_float(a[j]));
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (j < n_valid) red_add_f32(qrow + j * HD, __uint_as_float(a[j]));
      }
    }
    if (ok) ok = mbar_wait(done, 0, abort_flag);
    if (ok) {
      tc_fence_after();
      // warps 0-7 write dV, warps 8-15 write dK (scaled); the two warps of a lane quarter take 64 columns each
      const uint32_t tAcc = tmem_base + 256 + u * 128 + lane_off;
      const float mul = (u == 0) ? 1.f : scale;
      bf16* base = (u == 0) ? dV : dK;
      bf16* orow = base + (((size_t)b * Skv + kv_row) * H + h) * HD;
#pragma unroll 1
      for (int c = half * 2; c < half * 2 + 2; ++c) {
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
      atomicCAS(err, 0, 43);
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

// dq[b, s, h, :] = bf16(acc[b, h, s, :] * scale)
__global__ void __launch_bounds__(256) fa_bwd_dq_convert_kernel(const float* __restrict__ acc, bf16* __restrict__ dq, int B, int S, int H,
                                                                 float scale) {
  const long n8 = (long)B * S * H * 16;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n8; i += (long)gridDim.x * blockDim.x) {
    const int c = (int)(i & 15);
    const long row = i >> 4;             // over (b, s, h)
    const int h = (int)(row % H);
    const long bs = row / H;
    const int s_ = (int)(bs % S);
    const long b = bs / S;
    const float4* src = reinterpret_cast<const float4*>(acc + (((size_t)b * H + h) * S + s_) * 128 + c * 8);
    const float4 a = src[0], e = src[1];
    uint4 o;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
    o2[0] = __floats2bfloat162_rn(a.x * scale, a.y * scale);
    o2[1] = __floats2bfloat162_rn(a.z * scale, a.w * scale);
    o2[2] = __floats2bfloat162_rn(e.x * scale, e.y * scale);
    o2[3] = __floats2bfloat162_rn(e.z * scale, e.w * scale);
    reinterpret_cast<uint4*>(dq)[i] = o;
  }
}

}  // namespace cb200

using namespace cb200;

extern "C" void cb200_fa_bwd_dq_convert(const float* acc, void* dq, int B, int S, int H, float scale, cudaStream_t st) {
  const long n8 = (long)B * S * H * 16;
  fa_bwd_dq_convert_kernel<<<(unsigned)std::min<long>((n8 + 255) / 256, 148 * 16), 256, 0, st>>>(acc, (bf16*)dq, B, S, H, scale);
}

// Runs after the preprocessing kernel has produced lse2 / delta (padded to S_pad rows per (b, h)).
// dq_acc: B*Sq*H*128 floats of scratch, zeroed here.
extern "C" int cb200_fa_bwd_fused_main(const void* d_o, const void* q, const void* k, const void* v, const float* lse2,
                                       const float* delta, float* dq_acc, void* dq, void* dk, void* dv, int B, int Sq, int Skv, int H,
                                       int S_pad, float scale, int dbg, int* err, cudaStream_t st) {
  using namespace faf;
  (void)dbg;
  auto make = [&](CUtensorMap* m, const void* p, int S, int box_rows) {
    const uint64_t dims[4] = {(uint64_t)HD, (uint64_t)H, (uint64_t)S, (uint64_t)B};
    const uint64_t strides[3] = {(uint64_t)HD * 2, (uint64_t)H * HD * 2, (uint64_t)S * H * HD * 2};
    const uint32_t box[4] = {64, 1, (uint32_t)box_rows, 1};
    return make_tmap_bf16(m, p, 4, dims, strides, box);
  };
  CUtensorMap q64, do64, k128, v128;
  int rc = make(&q64, q, Sq, 64) | make(&do64, d_o, Sq, 64) | make(&k128, k, Skv, 128) | make(&v128, v, Skv, 128);
  if (rc) return rc;
  static bool attr = false;
  if (!attr) {
    cudaError_t e = cudaFuncSetAttribute(fa_bwd_fused_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmem);
    if (e != cudaSuccess) return 300 + (int)e;
    attr = true;
  }
  const size_t n = (size_t)B * Sq * H * HD;
  cudaError_t e = cudaMemsetAsync(dq_acc, 0, n * sizeof(float), st);
  if (e != cudaSuccess) return 400 + (int)e;
  dim3 grid((Skv + 127) / 128, H, B);
  fa_bwd_fused_kernel<<<grid, kThreads, kSmem, st>>>(q64, do64, k128, v128, lse2, delta, dq_acc, (bf16*)dk, (bf16*)dv, Sq, Skv, H, S_pad,
                                                     scale, err);
  const long n8 = (long)(n / 8);
  fa_bwd_dq_convert_kernel<<<(unsigned)std::min<long>((n8 + 255) / 256, 148 * 16), 256, 0, st>>>(dq_acc, (bf16*)dq, B, Sq, H, scale);
  return (int)cudaGetLastError();
}
