// Forward-mode (JVP) flash attention on tcgen05 / TMEM (sm_100a), head_dim 128, bf16, non-causal.
//
// Given the primal inputs q, k, v, their tangents tq, tk, tv, and the primal output o with its log-sum-exp (from the
// forward kernel), computes the tangent of the output
//
//     to = sum_j [ (P o tS) V + P tV ]  -  rowsum(P o tS) o o ,      tS = (tq k^T + q tk^T) * scale ,  P = softmax(q k^T * scale)
//
// in one pass over the keys. Because the log-sum-exp is known, P = exp2(S * c - lse * log2 e) is already normalised: no
// running maximum, no rescaling, and the two element-wise groups that alternate over key tiles never exchange state.
//
// A CTA owns one tile of 128 queries (Q and tQ resident in shared memory, a TMEM lane is a query row) and streams the keys
// in sub-tiles of 64. Per sub-tile:
//     S  = Q K^T                       (SS MMAs 128 x 64 x 128)
//     tS = tQ K^T + Q tK^T             (two accumulating SS MMA chains)
//     P, A = P o tS * scale            (element-wise warps; bf16 results written into TMEM over the fp32 tiles)
//     OT += A V + P tV                 (TS MMAs 128 x 128 x 64, V / tV read N-major)
// TMEM: buffer u in {0,1} at u*128: S [0,64), tS [64,128) (P bf16 -> [0,32), A bf16 -> [64,96)); OT = [256,384).
// The rank-one correction rowsum(A) o o is applied when OT is read out.
//
// Parity: replaces the Triton kernel of the reference (cosmos_predict2/_src/predict2/utils/flash_attention_jvp_triton.py:47-520).
// All waits are bounded and report through `err`.

#include <math.h>

#include "common.cuh"
#include "launchers.h"
#include "sm100.cuh"
#include "tmap.h"

namespace cb200 {
using namespace sm100;

namespace fj {
constexpr int HD = 128;
constexpr int kBig = 128 * HD * 2;    // 32 KB: 128-row tile
constexpr int kSmall = 64 * HD * 2;   // 16 KB: 64-row tile
constexpr int kThreads = 320;
constexpr int kMmaWarp = 9, kTmaWarp = 8;
constexpr int kRing = 8;              // K_j tK_j V_j tV_j of two sub-tiles
constexpr size_t kSmem = 2 * (size_t)kBig + kRing * (size_t)kSmall + 1024 + 1024 + 256;
}  // namespace fj

__device__ __forceinline__ float ex2j(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__global__ void __launch_bounds__(fj::kThreads, 1)
fa_jvp_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_tq,
              const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_tk,
              const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_tv,
              const bf16* __restrict__ O, const float* __restrict__ lse, bf16* __restrict__ TO, int Sq, int Skv, int H, float scale,
              int* __restrict__ err) {
  using namespace fj;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = smem;
  uint8_t* sTQ = smem + kBig;
  uint8_t* sR = smem + 2 * kBig;                       // ring: K_0 tK_0 V_0 tV_0 K_1 ...
  float* sMu = reinterpret_cast<float*>(sR + kRing * kSmall);   // [2 groups][128 rows]
  uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(sMu) + 1024);
  uint64_t* q_full = bars;
  uint64_t* r_full = bars + 1;
  uint64_t* r_empty = r_full + kRing;
  uint64_t* s_full = r_empty + kRing;   // [2]
  uint64_t* p_ready = s_full + 2;       // [2]
  uint64_t* done = p_ready + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(done + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;
  const int h = blockIdx.y, b = blockIdx.z;
  const int q_base = blockIdx.x * 128;
  const int n_kv = (Skv + 63) / 64;
  const float scale_log2 = scale * 1.4426950408889634f;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < kRing; ++i) {
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

  if (warp == kTmaWarp) {
    if (lane == 0) {
      prefetch_tmap(&tm_q);
      prefetch_tmap(&tm_tq);
      prefetch_tmap(&tm_k);
      prefetch_tmap(&tm_tk);
      prefetch_tmap(&tm_v);
      prefetch_tmap(&tm_tv);
      mbar_arrive_expect_tx(q_full, 2 * kBig);
      for (int c = 0; c < 2; ++c) {
        tma_load_4d(sQ + c * (kBig / 2), &tm_q, q_full, c * 64, h, q_base, b);
        tma_load_4d(sTQ + c * (kBig / 2), &tm_tq, q_full, c * 64, h, q_base, b);
      }
      bool ok = true;
      int slot = 0;
      uint32_t ph = 0;
      for (int n = 0; n < 4 * n_kv; ++n) {   // item n: sub-tile n/4, kind n%4 = K, tK, V, tV
        if (!mbar_wait(&r_empty[slot], ph ^ 1, abort_flag)) { ok = false; break; }
        mbar_arrive_expect_tx(&r_full[slot], kSmall);
        const int kind = n & 3;
        const CUtensorMap* tm = kind == 0 ? &tm_k : kind == 1 ? &tm_tk : kind == 2 ? &tm_v : &tm_tv;
        for (int c = 0; c < 2; ++c) tma_load_4d(sR + slot * kSmall + c * (kSmall / 2), tm, &r_full[slot], c * 64, h, (n >> 2) * 64, b);
        if (++slot == kRing) { slot = 0; ph ^= 1; }
      }
      if (!ok) { atomicCAS(err, 0, 51); *abort_flag = 1; }
    }
  } else if (warp == kMmaWarp) {
    // whole warp, warp-uniform values, elected lane issues
    const uint32_t leader = elect_one() ? 1u : 0u;
    auto wait_all = [&](uint64_t* bar, uint32_t parity) -> bool { return __all_sync(0xffffffffu, mbar_wait(bar, parity, abort_flag)); };
    constexpr uint32_t idesc_s = umma_idesc_bf16(128, 64, 0, 0);
    constexpr uint32_t idesc_o = umma_idesc_bf16(128, 128, 0, 1);
    const uint64_t dQ_km = umma_desc_sw128(smem_u32(sQ), 16, 1024);
    const uint64_t dTQ_km = umma_desc_sw128(smem_u32(sTQ), 16, 1024);
    const uint64_t dR_km = umma_desc_sw128(smem_u32(sR), 16, 1024);
    const uint64_t dR_mn = umma_desc_sw128(smem_u32(sR), kSmall / 2, 1024);
    // scores of sub-tile j into buffer u; the ring holds K_j at slot (4j) % 8 and tK_j right after it
    auto issue_scores = [&](int u, int k_slot, int tk_slot) {
      const uint64_t bk = dR_km + (uint64_t)(k_slot * (kSmall >> 4)), btk = dR_km + (uint64_t)(tk_slot * (kSmall >> 4));
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        const uint32_t offa = ((kk >> 2) * (kBig / 2) + (kk & 3) * 32) >> 4, offb = ((kk >> 2) * (kSmall / 2) + (kk & 3) * 32) >> 4;
        umma_ss_w(tmem_base + u * 128, dQ_km + offa, bk + offb, idesc_s, kk > 0 ? 1u : 0u, leader);
      }
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        const uint32_t offa = ((kk >> 2) * (kBig / 2) + (kk & 3) * 32) >> 4, offb = ((kk >> 2) * (kSmall / 2) + (kk & 3) * 32) >> 4;
        umma_ss_w(tmem_base + u * 128 + 64, dTQ_km + offa, bk + offb, idesc_s, kk > 0 ? 1u : 0u, leader);
      }
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        const uint32_t offa = ((kk >> 2) * (kBig / 2) + (kk & 3) * 32) >> 4, offb = ((kk >> 2) * (kSmall / 2) + (kk & 3) * 32) >> 4;
        umma_ss_w(tmem_base + u * 128 + 64, dQ_km + offa, btk + offb, idesc_s, 1u, leader);
      }
    };
    auto issue_out = [&](int u, int v_slot, int tv_slot, bool accumulate) {
      const uint64_t bv = dR_mn + (uint64_t)(v_slot * (kSmall >> 4)), btv = dR_mn + (uint64_t)(tv_slot * (kSmall >> 4));
#pragma unroll
      for (int kk = 0; kk < 4; ++kk)   // OT += A V
        umma_ts_w(tmem_base + 256, tmem_base + u * 128 + 64 + kk * 8, bv + (uint32_t)(kk * (2048 >> 4)), idesc_o,
                  (accumulate || kk > 0) ? 1u : 0u, leader);
#pragma unroll
      for (int kk = 0; kk < 4; ++kk)   // OT += P tV
        umma_ts_w(tmem_base + 256, tmem_base + u * 128 + kk * 8, btv + (uint32_t)(kk * (2048 >> 4)), idesc_o, 1u, leader);
    };
    bool ok = wait_all(q_full, 0);
    int slot = 0;
    uint32_t ph = 0;
    auto take = [&](int& out_slot) -> bool {
      if (!wait_all(&r_full[slot], ph)) return false;
      out_slot = slot;
      if (++slot == kRing) { slot = 0; ph ^= 1; }
      return true;
    };
    // ring order is K tK V tV per sub-tile, so the cursor must be advanced in that order: scores of sub-tile j+1 can only
    // be issued after the V / tV slots of sub-tile j have been taken
    int ks = 0, tks = 0, vs[2] = {0, 0}, tvs[2] = {0, 0};
    if (ok && n_kv > 0) {
      ok = take(ks) && take(tks);
      if (ok) {
        tc_fence_after();
        issue_scores(0, ks, tks);
        umma_commit_w(&r_empty[ks], leader);
        umma_commit_w(&r_empty[tks], leader);
        umma_commit_w(&s_full[0], leader);
      }
    }
    for (int j = 0; j < n_kv && ok; ++j) {
      const int u = j & 1;
      ok = take(vs[u]) && take(tvs[u]);
      if (!ok) break;
      if (j + 1 < n_kv) {   // scores of the next sub-tile go to the other buffer while this one is in the element-wise pass
        ok = take(ks) && take(tks);
        if (!ok) break;
        // buffer u^1 was last read by the output MMAs of sub-tile j-1, which precede these in issue order
        tc_fence_after();
        issue_scores(u ^ 1, ks, tks);
        umma_commit_w(&r_empty[ks], leader);
        umma_commit_w(&r_empty[tks], leader);
        umma_commit_w(&s_full[u ^ 1], leader);
      }
      if (!wait_all(&p_ready[u], (j >> 1) & 1)) { ok = false; break; }
      tc_fence_after();
      issue_out(u, vs[u], tvs[u], j > 0);
      umma_commit_w(&r_empty[vs[u]], leader);
      umma_commit_w(&r_empty[tvs[u]], leader);
    }
    if (ok) umma_commit_w(done, leader);
    if (!ok && lane == 0) { atomicCAS(err, 0, 52); *abort_flag = 1; }
  } else {
    // ------------------------------------------------------------------ element-wise groups (group u owns buffer u)
    const int u = warp >> 2, quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const int q_row = q_base + row;
    const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
    const uint32_t tS = tmem_base + u * 128 + lane_off;
    const uint32_t tTS = tS + 64;
    const size_t bh = (size_t)b * H + h;
    const float nlse2 = (q_row < Sq) ? -lse[bh * Sq + q_row] * 1.4426950408889634f : -INFINITY;   // -inf: rows past the end give P = 0
    float mu = 0.f;
    bool ok = true;
    for (int j = u; j < n_kv; j += 2) {
      if (!mbar_wait(&s_full[u], (j >> 1) & 1, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const int kv0 = j * 64;
      const bool ragged = kv0 + 64 > Skv;
      uint32_t pp[2][16], pa[2][16];
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t s[32], ts[32];
        tmem_ld32(tS + c * 32, s);
        tmem_ld32(tTS + c * 32, ts);
        tmem_ld_wait();
#pragma unroll
        for (int g = 0; g < 16; ++g) {
          float p0 = ex2j(fmaf(__uint_as_float(s[2 * g]), scale_log2, nlse2));
          float p1 = ex2j(fmaf(__uint_as_float(s[2 * g + 1]), scale_log2, nlse2));
          if (ragged) {
            if (kv0 + c * 32 + 2 * g >= Skv) p0 = 0.f;
            if (kv0 + c * 32 + 2 * g + 1 >= Skv) p1 = 0.f;
          }
          const float a0 = p0 * (__uint_as_float(ts[2 * g]) * scale), a1 = p1 * (__uint_as_float(ts[2 * g + 1]) * scale);
          mu += a0 + a1;
          __nv_bfloat162 pb = __floats2bfloat162_rn(p0, p1), ab = __floats2bfloat162_rn(a0, a1);
          pp[c][g] = *reinterpret_cast<uint32_t*>(&pb);
          pa[c][g] = *reinterpret_cast<uint32_t*>(&ab);
        }
      }
      // both fp32 tiles of this row have been read: P -> [0,32), A -> [64,96)
      tmem_st16(tS, pp[0]);
      tmem_st16(tS + 16, pp[1]);
      tmem_st16(tTS, pa[0]);
      tmem_st16(tTS + 16, pa[1]);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_ready[u]);
    }
    sMu[u * 128 + row] = mu;
    asm volatile("bar.sync 1, 256;" ::: "memory");   // the eight element-wise warps
    const float mu_all = sMu[row] + sMu[128 + row];
    if (ok) ok = mbar_wait(done, 0, abort_flag);
    if (ok) {
      tc_fence_after();
      // group 0 reads out columns [0,64), group 1 [64,128):  to = OT - mu * o
      const uint32_t tAcc = tmem_base + 256 + u * 64 + lane_off;
      const size_t goff = (((size_t)b * Sq + q_row) * H + h) * HD + u * 64;
#pragma unroll 1
      for (int c = 0; c < 2; ++c) {
        uint32_t o[32];
        tmem_ld32(tAcc + c * 32, o);
        tmem_ld_wait();
        if (q_row < Sq) {
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            const uint4 ov = *reinterpret_cast<const uint4*>(O + goff + c * 32 + q4 * 8);
            const __nv_bfloat162* o2 = reinterpret_cast<const __nv_bfloat162*>(&ov);
            uint4 rv;
            __nv_bfloat162* r2 = reinterpret_cast<__nv_bfloat162*>(&rv);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 of = __bfloat1622float2(o2[e]);
              r2[e] = __floats2bfloat162_rn(__uint_as_float(o[q4 * 8 + 2 * e]) - mu_all * of.x,
                                            __uint_as_float(o[q4 * 8 + 2 * e + 1]) - mu_all * of.y);
            }
            *reinterpret_cast<uint4*>(TO + goff + c * 32 + q4 * 8) = rv;
          }
        }
      }
    } else if (lane == 0) {
      atomicCAS(err, 0, 53);
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

// q, tq, o, to [B,Sq,H,128]; k, tk, v, tv [B,Skv,H,128]; lse [B,H,Sq] (natural log) from the forward kernel
extern "C" int cb200_fa_jvp(const void* q, const void* k, const void* v, const void* tq, const void* tk, const void* tv, const void* o,
                            const float* lse, void* to, int B, int Sq, int Skv, int H, float scale, int* err, cudaStream_t st) {
  using namespace fj;
  auto make = [&](CUtensorMap* m, const void* p, int S, int box_rows) {
    const uint64_t dims[4] = {(uint64_t)HD, (uint64_t)H, (uint64_t)S, (uint64_t)B};
    const uint64_t strides[3] = {(uint64_t)HD * 2, (uint64_t)H * HD * 2, (uint64_t)S * H * HD * 2};
    const uint32_t box[4] = {64, 1, (uint32_t)box_rows, 1};
    return make_tmap_bf16(m, p, 4, dims, strides, box);
  };
  CUtensorMap mq, mtq, mk, mtk, mv, mtv;
  int rc = make(&mq, q, Sq, 128) | make(&mtq, tq, Sq, 128) | make(&mk, k, Skv, 64) | make(&mtk, tk, Skv, 64) | make(&mv, v, Skv, 64) |
           make(&mtv, tv, Skv, 64);
  if (rc) return rc;
  static bool attr = false;
  if (!attr) {
    cudaError_t e = cudaFuncSetAttribute(fa_jvp_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmem);
    if (e != cudaSuccess) return 500 + (int)e;
    attr = true;
  }
  dim3 grid((Sq + 127) / 128, H, B);
  fa_jvp_kernel<<<grid, kThreads, kSmem, st>>>(mq, mtq, mk, mtk, mv, mtv, (const bf16*)o, lse, (bf16*)to, Sq, Skv, H, scale, err);
  return (int)cudaGetLastError();
}
