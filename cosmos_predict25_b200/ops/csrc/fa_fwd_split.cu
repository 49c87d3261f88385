// Flash attention forward on tcgen05 / TMEM (sm_100a), head_dim 128, bf16, non-causal: the variant with TWO threads per
// query row.
//
// Same pipeline as fa_fwd.cu (two 128-row query tiles per CTA ping-pong through S/O TMEM buffers, one TMA warp, one MMA
// warp, P written back into TMEM as bf16 and consumed by a TS MMA), but every query tile is served by eight softmax
// warps instead of four: warps w and w + 4 of a tile own the same 32 TMEM lanes (rows) and split the 128 key columns
// in halves. The exponentials of one row (the MUFU-serial part of the S -> P -> O dependency chain) then take half as
// long, which is what bounds the single-thread-per-row kernel. The two threads of a row agree on the row maximum through
// a 1 KB shared-memory table (bf16, rounded up: the reference maximum only has to be common and not smaller than the true
// one) and a 64-thread named barrier per kv tile; their partial row sums are only combined at the end.
//
//   warps 0-7   softmax of query tile 0: quarter = w & 3 (TMEM lanes), half = (w >> 2) & 1 (key columns)
//   warps 8-15  softmax of query tile 1
//   warp  16    TMA producer
//   warp  17    MMA issuer
//
// Measured on a B200 at S = 84,480, H = 16: 53.7 ms against 48.5 ms for the one-thread-per-row kernel, which therefore
// stays the default; this variant is reachable as variant 6 of the forward operator and is kept tested.
//
// Hazard that fixes the order of operations: P (bf16) overwrites S columns [0, 64), which are the scores of keys 0..63,
// i.e. of half 0.  Half 0 therefore keeps its 64 scores in registers, and nobody stores P before the pair barrier that
// follows both halves' loads.

#include <math.h>

#include "common.cuh"
#include "launchers.h"
#include "sm100.cuh"
#include "tmap.h"

namespace cb200 {
using namespace sm100;

namespace fas {
constexpr int HD = 128;
constexpr int BQ = 128;
constexpr int BKV = 128;
constexpr int kTileBytes = 128 * HD * 2;
constexpr int kHalfBytes = kTileBytes / 2;
constexpr int kRing = 5;
constexpr int kThreads = 576;
constexpr int kMmaWarp = 17, kTmaWarp = 16;
constexpr int kXchBytes = 1024;  // [2 tiles][2 halves][128 rows] bf16 row maxima; reused as [2][128] fp32 row sums at the end
constexpr size_t kSmem = (2 + kRing) * (size_t)kTileBytes + 1024 + 256 + kXchBytes;
constexpr float kRescaleThreshold = 8.0f;
}  // namespace fas

__device__ __forceinline__ float ex2s(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ void pair_barrier(int id) { asm volatile("bar.sync %0, 64;" ::"r"(id) : "memory"); }

struct SeqScatterS {
  int64_t ptrs[8];
  int P, rank, S_loc;
};

__global__ void __maxnreg__(96)
fa_fwd_split_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
              const __grid_constant__ CUtensorMap tm_v, bf16* __restrict__ O, float* __restrict__ LSE, int Sq, int Skv, int H,
              float scale_log2, SeqScatterS sc, int* __restrict__ err) {
  using namespace fas;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = smem;                     // 2 tiles
  uint8_t* sR = smem + 2 * kTileBytes;    // ring of kRing tiles: K_0 V_0 K_1 V_1 ...
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (2 + kRing) * kTileBytes);
  uint64_t* q_full = bars;                 // [1]
  uint64_t* r_full = bars + 1;             // [kRing]
  uint64_t* r_empty = bars + 1 + kRing;    // [kRing]
  uint64_t* s_full = bars + 1 + 2 * kRing; // [2]  scores of tile t ready (also: all earlier MMAs complete)
  uint64_t* p_ready = s_full + 2;          // [2]  probabilities of tile t written to TMEM
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(p_ready + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  uint8_t* xch = smem + (2 + kRing) * kTileBytes + 256;  // row maxima / row sums exchanged between the two threads of a row

  // the shuffle makes the warp index (and every role branch below) provably warp-uniform for the compiler
  const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;
  const int h = blockIdx.y, b = blockIdx.z;
  const int q_base = blockIdx.x * 2 * BQ;
  const int n_kv = (Skv + BKV - 1) / BKV;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < kRing; ++i) {
      mbar_init(&r_full[i], 1);
      mbar_init(&r_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&p_ready[i], 8);
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

  if (warp == kTmaWarp) {
    // -------------------------------------------------------------------- TMA producer
    if (lane == 0) {
      prefetch_tmap(&tm_q);
      prefetch_tmap(&tm_k);
      prefetch_tmap(&tm_v);
      mbar_arrive_expect_tx(q_full, 2 * kTileBytes);
      for (int t = 0; t < 2; ++t)
        for (int c = 0; c < 2; ++c)
          tma_load_4d(sQ + t * kTileBytes + c * kHalfBytes, &tm_q, q_full, c * 64, h, q_base + t * BQ, b);
      bool ok = true;
      int slot = 0;
      uint32_t ph = 0;
      for (int n = 0; n < 2 * n_kv; ++n) {  // even n: K_{n/2}, odd n: V_{n/2}
        if (!mbar_wait(&r_empty[slot], ph ^ 1, abort_flag)) { ok = false; break; }
        mbar_arrive_expect_tx(&r_full[slot], kTileBytes);
        const CUtensorMap* tm = (n & 1) ? &tm_v : &tm_k;
        const int kv_tile = n >> 1;
        for (int c = 0; c < 2; ++c) tma_load_4d(sR + slot * kTileBytes + c * kHalfBytes, tm, &r_full[slot], c * 64, h, kv_tile * BKV, b);
        if (++slot == kRing) { slot = 0; ph ^= 1; }
      }
      if (!ok) { atomicCAS(err, 0, 11); *abort_flag = 1; }
    }
  } else if (warp == kMmaWarp) {
    // -------------------------------------------------------------------- MMA issuer
    {
      // The whole warp runs this code with identical values and only the elected lane issues: warp-uniform control flow
      // and descriptor arithmetic stay on the uniform datapath, which roughly halves the issue cost per MMA.
      const uint32_t leader = elect_one() ? 1u : 0u;
      auto wait_all = [&](uint64_t* bar, uint32_t parity) -> bool { return __all_sync(0xffffffffu, mbar_wait(bar, parity, abort_flag)); };
      constexpr uint32_t idesc_qk = umma_idesc_bf16(128, 128, 0, 0);
      constexpr uint32_t idesc_pv = umma_idesc_bf16(128, 128, 0, 1);
      bool ok = wait_all(q_full, 0);
      const uint64_t dQ_km = umma_desc_sw128(smem_u32(sQ), 16, 1024);          // Q tiles as K-major A
      const uint64_t dR_km = umma_desc_sw128(smem_u32(sR), 16, 1024);          // ring slot as K-major B (K)
      const uint64_t dR_mn = umma_desc_sw128(smem_u32(sR), kHalfBytes, 1024);  // ring slot as N-major B (V)
      auto issue_qk = [&](int t, int slot) {
        const uint64_t bq = dQ_km + (uint64_t)(t * (kTileBytes >> 4)), bk = dR_km + (uint64_t)(slot * (kTileBytes >> 4));
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t off = ((kk >> 2) * kHalfBytes + (kk & 3) * 32) >> 4;
          umma_ss_w(tmem_base + t * 128, bq + off, bk + off, idesc_qk, kk > 0 ? 1u : 0u, leader);
        }
      };
      auto issue_pv = [&](int t, int slot, bool accumulate) {
        const uint64_t bv = dR_mn + (uint64_t)(slot * (kTileBytes >> 4));
#pragma unroll
        for (int kk = 0; kk < BKV / 16; ++kk) {
          umma_ts_w(tmem_base + 256 + t * 128, tmem_base + t * 128 + kk * 8, bv + (uint32_t)(kk * (2048 >> 4)), idesc_pv,
                    (accumulate || kk > 0) ? 1u : 0u, leader);
        }
      };
      // ring cursor of the item to consume next (K_0 first)
      int slot = 0;
      uint32_t ph = 0;
      auto advance = [&]() { if (++slot == kRing) { slot = 0; ph ^= 1; } };
      if (ok) ok = wait_all(&r_full[slot], ph);
      if (ok) {
        tc_fence_after();
        issue_qk(0, slot);
        umma_commit_w(&s_full[0], leader);
        issue_qk(1, slot);
        umma_commit_w(&s_full[1], leader);
        umma_commit_w(&r_empty[slot], leader);
        advance();
      }
      for (int j = 0; j < n_kv && ok; ++j) {
        const bool has_next = (j + 1) < n_kv;
        const int v_slot = slot;
        if (!wait_all(&r_full[v_slot], ph)) { ok = false; break; }
        advance();
        const int k_slot = slot;
        if (has_next) {
          if (!wait_all(&r_full[k_slot], ph)) { ok = false; break; }
          advance();
        }
        for (int t = 0; t < 2; ++t) {
          if (!wait_all(&p_ready[t], j & 1)) { ok = false; break; }
          tc_fence_after();
          issue_pv(t, v_slot, j > 0);
          if (t == 1) umma_commit_w(&r_empty[v_slot], leader);
          if (has_next) issue_qk(t, k_slot);
          if (t == 1 && has_next) umma_commit_w(&r_empty[k_slot], leader);
          umma_commit_w(&s_full[t], leader);
        }
      }
      if (!ok && lane == 0) { atomicCAS(err, 0, 12); *abort_flag = 1; }
    }
  } else {
    // -------------------------------------------------------------------- softmax warps (two threads per row)
    const int t = warp >> 3;            // query tile
    const int half = (warp >> 2) & 1;   // key columns [64 * half, 64 * half + 64)
    const int quarter = warp & 3;       // TMEM lane quarter
    const int row = quarter * 32 + lane;
    const int q_row = q_base + t * BQ + row;
    const int bar_id = 1 + t * 4 + quarter;
    const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
    const uint32_t tS = tmem_base + t * 128 + lane_off;
    const uint32_t tO = tmem_base + 256 + t * 128 + lane_off;
    __nv_bfloat16* xmax = reinterpret_cast<__nv_bfloat16*>(xch) + t * 256;   // [2 halves][128 rows]
    float m_ref = -INFINITY;
    float l = 0.f;                      // partial row sum over this thread's key columns
    bool ok = true;
    for (int j = 0; j < n_kv; ++j) {
      // A warp whose wait ran out keeps walking through the pair barriers (without touching TMEM) so that its partner,
      // which may have passed the same wait a moment earlier, is never left alone at one.
      if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&s_full[t], j & 1, abort_flag));
      uint32_t r[2][32];
      __nv_bfloat16 mine = __float2bfloat16(0.f);
      if (ok) {
        tc_fence_after();
        tmem_ld32(tS + half * 64, r[0]);
        tmem_ld32(tS + half * 64 + 32, r[1]);
        tmem_ld_wait();
        const int n_valid = Skv - j * BKV - half * 64;
        if (n_valid < 64) {
#pragma unroll
          for (int c = 0; c < 2; ++c)
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (c * 32 + i >= n_valid) r[c][i] = 0xff800000u;  // -inf
        }
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int c = 0; c < 2; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(r[c][i]));
        // both threads of the row use the rounded-up bf16 values, their own included, so they always agree
        mine = __float2bfloat16_ru(fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * scale_log2);
        xmax[half * 128 + row] = mine;
      }
      pair_barrier(bar_id);             // also orders: every S load of the row is done before any P store below
      if (!ok) continue;
      const float mx = fmaxf(__bfloat162float(mine), __bfloat162float(xmax[(half ^ 1) * 128 + row]));
      const bool need = mx > m_ref + kRescaleThreshold;
      float alpha = 1.f;
      if (need) {
        alpha = (m_ref == -INFINITY) ? 0.f : ex2s(m_ref - mx);
        m_ref = mx;
        l *= alpha;
      }
      const bool rescale = j > 0 && __any_sync(0xffffffffu, need);
      const float neg_m = -m_ref;
      float2 lsum2 = make_float2(0.f, 0.f);
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float px = ex2s(fmaf(__uint_as_float(r[c][2 * i]), scale_log2, neg_m));
          const float py = ex2s(fmaf(__uint_as_float(r[c][2 * i + 1]), scale_log2, neg_m));
          lsum2.x += px;
          lsum2.y += py;
          __nv_bfloat162 pb = __floats2bfloat162_rn(px, py);
          pk[i] = *reinterpret_cast<uint32_t*>(&pb);
        }
        tmem_st16(tS + half * 32 + c * 16, pk);   // keys 64*half + 32*c + [0, 32) -> packed columns 32*half + 16*c + [0, 16)
      }
      l += lsum2.x + lsum2.y;
      if (rescale) {
        // rescale this thread's 64 output columns in TMEM (after the probabilities: the score registers are free by now)
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t o[16];
          tmem_ld16(tO + half * 64 + c * 16, o);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tmem_st16(tO + half * 64 + c * 16, o);
        }
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_ready[t]);
    }
    if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&s_full[t], n_kv & 1, abort_flag));
    // combine the two partial row sums (the table of maxima is free now: every read of it precedes the last p_ready arrival)
    float* xsum = reinterpret_cast<float*>(xch) + t * 128;
    if (half == 1) xsum[row] = l;
    pair_barrier(bar_id);
    if (half == 0) {
      l += xsum[row];
      xsum[row] = l;
    }
    pair_barrier(bar_id);
    if (half == 1) l = xsum[row];
    if (ok) {
      tc_fence_after();
      const float inv_l = 1.f / l;
      bf16* orow = O + (((size_t)b * Sq + q_row) * H + h) * HD;
      if (sc.P > 0 && q_row < Sq) {
        const int dst = q_row / sc.S_loc, s_loc = q_row - dst * sc.S_loc;
        orow = reinterpret_cast<bf16*>(sc.ptrs[dst]) + (((size_t)b * sc.S_loc + s_loc) * (sc.P * H) + sc.rank * H + h) * HD;
      }
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t o[16];
        tmem_ld16(tO + half * 64 + c * 16, o);
        tmem_ld_wait();
        if (q_row < Sq) {
#pragma unroll
          for (int q = 0; q < 2; ++q) {
            uint4 ov;
            __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
            for (int i = 0; i < 4; ++i)
              o2[i] = __floats2bfloat162_rn(__uint_as_float(o[q * 8 + 2 * i]) * inv_l, __uint_as_float(o[q * 8 + 2 * i + 1]) * inv_l);
            *reinterpret_cast<uint4*>(orow + half * 64 + c * 16 + q * 8) = ov;
          }
        }
      }
      if (half == 0 && q_row < Sq) LSE[((size_t)b * H + h) * Sq + q_row] = (m_ref + log2f(l)) * 0.6931471805599453f;
    } else if (lane == 0) {
      atomicCAS(err, 0, 13);
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

// q [B, Sq, H, 128]; k, v [B, Skv, H, 128]; o like q; lse [B, H, Sq] fp32.  out_ptrs != nullptr: rows are scattered to the
// P ranks' sequence shards ([B, Sq / P, P*H, 128] on each) instead of being written to o.
extern "C" int cb200_fa_fwd_split(const void* q, const void* k, const void* v, void* o, float* lse, int B, int Sq, int Skv, int H,
                                  float scale, const int64_t* out_ptrs, int P, int rank, int* err, cudaStream_t st) {
  using namespace fas;
  CUtensorMap tq, tk, tv;
  auto make = [&](CUtensorMap* m, const void* p, int S) {
    const uint64_t dims[4] = {(uint64_t)HD, (uint64_t)H, (uint64_t)S, (uint64_t)B};
    const uint64_t strides[3] = {(uint64_t)HD * 2, (uint64_t)H * HD * 2, (uint64_t)S * H * HD * 2};
    const uint32_t box[4] = {64, 1, 128, 1};
    return make_tmap_bf16(m, p, 4, dims, strides, box);
  };
  int rc = make(&tq, q, Sq);
  if (rc) return rc;
  rc = make(&tk, k, Skv);
  if (rc) return rc;
  rc = make(&tv, v, Skv);
  if (rc) return rc;
  SeqScatterS sc{};
  if (out_ptrs != nullptr) {
    if (P < 1 || P > 8 || Sq % P != 0 || rank < 0 || rank >= P) return -21;
    for (int i = 0; i < P; ++i) sc.ptrs[i] = out_ptrs[i];
    sc.P = P;
    sc.rank = rank;
    sc.S_loc = Sq / P;
  }
  static bool attr = false;
  if (!attr) {
    cudaError_t e = cudaFuncSetAttribute(fa_fwd_split_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmem);
    if (e != cudaSuccess) return 100 + (int)e;
    attr = true;
  }
  dim3 grid((Sq + 2 * BQ - 1) / (2 * BQ), H, B);
  fa_fwd_split_kernel<<<grid, kThreads, kSmem, st>>>(tq, tk, tv, (bf16*)o, lse, Sq, Skv, H, scale * 1.4426950408889634f, sc, err);
  return (int)cudaGetLastError();
}
