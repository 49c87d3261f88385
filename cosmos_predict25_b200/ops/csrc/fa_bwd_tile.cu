// Flash attention backward, one pass over the score matrix in 128 x 128 tiles (5 GEMMs per tile, every MMA 128 x 128 x 16),
// tcgen05 / TMEM, sm_100a, head_dim 128, bf16, non-causal.
//
// A CTA owns one tile of 128 keys (K, V resident in shared memory, dK and dV accumulated in TMEM) and streams the queries in
// tiles of 128. It works on the transposed problem, so a TMEM lane is a key row:
//
//   S^T  = K Q^T            SS MMA -> X (TMEM, 128 fp32 columns)
//   dP^T = V dO^T           SS MMA -> Y (TMEM, 128 fp32 columns)
//   P^T  = exp2(S^T c - lse)                element-wise phase 1: X -> bf16 P^T written back into X
//   dV  += P^T dO           TS MMA (A = P^T from TMEM)
//   dS^T = P^T o (dP^T - delta)             element-wise phase 2: Y -> bf16 dS^T tile in shared memory
//   dQ^T = K^T dS^T         SS MMA -> Y (K read M-major, dS^T N-major), drained by four warps into an fp32 dQ buffer in global
//                           memory with red.global.add (a warp instruction = 32 consecutive d of one query = one 128-byte line)
//   dK  += dS^T Q           SS MMA (A = the same dS^T tile read K-major)
//
// Why this shape: with 64-query sub-tiles the N = 64 MMAs re-read their 4 KB A slice from shared memory every 32 tensor
// clocks, which exceeds the 128 B/clk a CTA's shared memory delivers; at N = 128 an SS MMA needs exactly 128 B/clk and a TS MMA
// half of that. X and Y are single buffers: the pipeline comes from splitting the element-wise work into the two phases above,
// each of which overlaps the MMAs that do not depend on it. In steady state the MMA warp issues, per query tile i,
//
//   [P^T(i) ready]  dV(i), S^T(i+1)   |   [dS^T(i) ready]  dQ^T(i), dK(i)   |   [dQ^T(i) drained]  dP^T(i+1)
//
// while the element-wise warps compute dS^T(i) (beside dV / S^T) and then P^T(i+1) (beside dQ^T / dK / dP^T), and the drain
// warps empty Y beside dK(i).
//
// Shared memory (7 tiles of 32 KB): K, V, three Q stages (a Q tile lives from S^T(i) to dK(i)), one dO stage (dP^T(i) to dV(i)),
// dS^T. Row statistics (-lse*log2e, -delta) travel in their own two-stage ring. All waits are bounded and report through `err`.
//
// Neighbourhood (tile-sparse) mode, template flag NA: the tensors arrive in tile order (every 128-row tile is one 4 x 4 x 8 box of
// video tokens, row = dt * 32 + dh * 8 + dw), a CTA walks the list of query tiles that see its key tile instead of all of them,
// and phase 1 clears the entries of P^T whose (key, query) pair is not visible: per axis a byte table indexed by
// (key coordinate, query tile) holds the visibility bits of the tile's 4 / 4 / 8 query coordinates, and a pair is visible when its
// three bits are set. Tiles that are visible as a whole (list entry with the top bit set) skip the masking.

#include <math.h>

#include <algorithm>

#include "common.cuh"
#include "launchers.h"
#include "sm100.cuh"
#include "tmap.h"

namespace cb200 {
using namespace sm100;

namespace fat {
constexpr int HD = 128;
constexpr int kTile = 128 * HD * 2;   // 32 KB
constexpr int kHalf = kTile / 2;      // one 64-column half: [128 rows][128 bytes], 128-byte swizzle
constexpr int kQStages = 3;
constexpr int kEwWarps = 16, kDrainWarps = 4;
constexpr int kTmaWarp = kEwWarps + kDrainWarps, kMmaWarp = kTmaWarp + 1;
constexpr int kThreads = (kMmaWarp + 1) * 32;   // 704
constexpr int kStatBytes = 1024;      // per stage: 128 (-lse*log2e) + 128 (-delta) floats
constexpr size_t kSmem = (size_t)(2 + kQStages + 1 + 1) * kTile + 2 * kStatBytes + 256;
constexpr uint32_t X = 0, Y = 128, DV = 256, DK = 384;   // TMEM columns
}  // namespace fat

struct NaBwdPlan {
  const int* q_list;       // [key tiles][max_n]: query tile index, top bit = the whole tile pair is visible
  const int* q_cnt;        // [key tiles]
  const uint8_t* bt;       // [T][nT], [H][nH], [W][nW]: visibility bits of a query tile's coordinates for one key coordinate
  const uint8_t* bh;
  const uint8_t* bw;
  int max_n, nT, nH, nW;
};

__device__ __forceinline__ float ex2t(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void red_add_f32t(float* p, float v) {
  asm volatile("red.global.add.f32 [%0], %1;" ::"l"(p), "f"(v) : "memory");
}

template <bool NA>
__global__ void __launch_bounds__(fat::kThreads, 1)
fa_bwd_tile_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_do,
                   const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                   const float* __restrict__ lse2, const float* __restrict__ delta, float* __restrict__ dQacc,
                   bf16* __restrict__ dK, bf16* __restrict__ dV, int Sq, int Skv, int H, int Sq_pad, float scale,
                   NaBwdPlan na, int* __restrict__ err) {
  using namespace fat;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* sK = smem;
  uint8_t* sV = smem + kTile;
  uint8_t* sQ = smem + 2 * kTile;                       // kQStages tiles
  uint8_t* sDO = sQ + kQStages * kTile;
  uint8_t* sDS = sDO + kTile;                           // dS^T [128 keys][128 queries] bf16, two 64-query halves
  float* sStat = reinterpret_cast<float*>(sDS + kTile);  // [2 stages][256]
  uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(sStat) + 2 * kStatBytes);
  uint64_t* kv_full = bars;              // [1]
  uint64_t* q_full = bars + 1;           // [3]
  uint64_t* q_empty = q_full + kQStages; // [3]
  uint64_t* do_full = q_empty + kQStages;
  uint64_t* do_empty = do_full + 1;
  uint64_t* st_full = do_empty + 1;      // [2]
  uint64_t* st_empty = st_full + 2;      // [2] 16 arrivals
  uint64_t* s_full = st_empty + 2;       // S^T in X
  uint64_t* p_ready = s_full + 1;        // P^T in X (16 arrivals)
  uint64_t* dp_full = p_ready + 1;       // dP^T in Y
  uint64_t* ds_ready = dp_full + 1;      // dS^T in shared memory, Y read (16 arrivals)
  uint64_t* dq_full = ds_ready + 1;      // dQ^T in Y
  uint64_t* dq_free = dq_full + 1;       // Y drained (4 arrivals)
  uint64_t* done = dq_free + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(done + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  // the shuffle makes the warp index (and every role branch below) provably warp-uniform for the compiler
  const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;
  const int h = blockIdx.y, b = blockIdx.z;
  const int kv_base = blockIdx.x * 128;
  // query tiles this CTA visits, and the tile index of visit i
  const int n_q = NA ? na.q_cnt[blockIdx.x] : (Sq + 127) / 128;
  const int* my_list = NA ? na.q_list + (size_t)blockIdx.x * na.max_n : nullptr;
  auto q_tile = [&](int i) -> int { return NA ? (my_list[i] & 0x7fffffff) : i; };
  const float scale_log2 = scale * 1.4426950408889634f;

  // The 128-byte swizzle of TMA and of the UMMA descriptors is a function of the shared-memory address, so every tile must
  // start on a 1024-byte boundary; the kernel has no static shared memory and takes the dynamic window's base as it is.
  if ((smem_u32(smem) & 1023u) != 0) {
    if (threadIdx.x == 0) atomicCAS(err, 0, 50);
    return;
  }
  // A CTA that starts after another one has reported an error leaves at once (the whole grid then drains in microseconds
  // instead of running every CTA into its own wait limit). One thread reads the word so that the decision is CTA-uniform.
  if (threadIdx.x == 0) *abort_flag = *reinterpret_cast<volatile int*>(err);
  __syncthreads();
  if (*abort_flag != 0) return;
  __syncthreads();
  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int i = 0; i < kQStages; ++i) {
      mbar_init(&q_full[i], 1);
      mbar_init(&q_empty[i], 1);
    }
    mbar_init(do_full, 1);
    mbar_init(do_empty, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&st_full[i], 1);
      mbar_init(&st_empty[i], kEwWarps);
    }
    mbar_init(s_full, 1);
    mbar_init(p_ready, kEwWarps);
    mbar_init(dp_full, 1);
    mbar_init(ds_ready, kEwWarps);
    mbar_init(dq_full, 1);
    mbar_init(dq_free, kDrainWarps);
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
    // ------------------------------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      prefetch_tmap(&tm_q);
      prefetch_tmap(&tm_do);
      prefetch_tmap(&tm_k);
      prefetch_tmap(&tm_v);
      mbar_arrive_expect_tx(kv_full, 2 * kTile);
      for (int c = 0; c < 2; ++c) {
        tma_load_4d(sK + c * kHalf, &tm_k, kv_full, c * 64, h, kv_base, b);
        tma_load_4d(sV + c * kHalf, &tm_v, kv_full, c * 64, h, kv_base, b);
      }
      bool ok = true;
      for (int i = 0; i < n_q && ok; ++i) {
        const int qs = i % kQStages, ss = i & 1;
        const int q0 = q_tile(i) * 128;
        if (!mbar_wait(&q_empty[qs], ((i / kQStages) & 1) ^ 1, abort_flag)) { ok = false; break; }
        mbar_arrive_expect_tx(&q_full[qs], kTile);
        for (int c = 0; c < 2; ++c) tma_load_4d(sQ + qs * kTile + c * kHalf, &tm_q, &q_full[qs], c * 64, h, q0, b);
        if (!mbar_wait(&st_empty[ss], ((i >> 1) & 1) ^ 1, abort_flag)) { ok = false; break; }
        mbar_arrive_expect_tx(&st_full[ss], kStatBytes);
        float* st = sStat + ss * 256;
        bulk_load_1d(st, lse2 + bh * Sq_pad + (size_t)q0, 512, &st_full[ss]);
        bulk_load_1d(st + 128, delta + bh * Sq_pad + (size_t)q0, 512, &st_full[ss]);
        if (!mbar_wait(do_empty, (i & 1) ^ 1, abort_flag)) { ok = false; break; }
        mbar_arrive_expect_tx(do_full, kTile);
        for (int c = 0; c < 2; ++c) tma_load_4d(sDO + c * kHalf, &tm_do, do_full, c * 64, h, q0, b);
      }
      if (!ok) { atomicCAS(err, 0, 51); *abort_flag = 1; }
    }
  } else if (warp == kMmaWarp) {
    // ------------------------------------------------------------------------------------------ MMA issuer
    // the whole warp runs this code with identical values; only `leader` issues (see umma_ss_w)
    const uint32_t leader = elect_one() ? 1u : 0u;
    auto wait_all = [&](uint64_t* bar, uint32_t parity) -> bool { return __all_sync(0xffffffffu, mbar_wait(bar, parity, abort_flag)); };
    constexpr uint32_t idesc_kk = umma_idesc_bf16(128, 128, 0, 0);   // A, B K-major
    constexpr uint32_t idesc_kn = umma_idesc_bf16(128, 128, 0, 1);   // B N-major
    constexpr uint32_t idesc_mn = umma_idesc_bf16(128, 128, 1, 1);   // A M-major, B N-major
    // Base descriptors are built once; an operand slice is the base plus a constant added to the address field (16-byte
    // units, no carry out of the field because shared memory is smaller than 256 KB).
    const uint64_t dK_km = umma_desc_sw128(smem_u32(sK), 16, 1024);       // K   as K-major A (S^T)
    const uint64_t dV_km = umma_desc_sw128(smem_u32(sV), 16, 1024);       // V   as K-major A (dP^T)
    const uint64_t dK_mn = umma_desc_sw128(smem_u32(sK), kHalf, 1024);    // K^T as M-major A (dQ^T)
    const uint64_t dQ_km = umma_desc_sw128(smem_u32(sQ), 16, 1024);       // Q stage as K-major B (S^T)
    const uint64_t dQ_mn = umma_desc_sw128(smem_u32(sQ), kHalf, 1024);    // Q stage as N-major B (dK)
    const uint64_t dDO_km = umma_desc_sw128(smem_u32(sDO), 16, 1024);     // dO as K-major B (dP^T)
    const uint64_t dDO_mn = umma_desc_sw128(smem_u32(sDO), kHalf, 1024);  // dO as N-major B (dV)
    const uint64_t dDS_km = umma_desc_sw128(smem_u32(sDS), 16, 1024);     // dS^T as K-major A (dK)
    const uint64_t dDS_mn = umma_desc_sw128(smem_u32(sDS), kHalf, 1024);  // dS^T as N-major B (dQ^T)
    // K-major operand, k-step kk of 16 elements: 32 bytes inside the 128-byte row, second 64-element half after 4 steps
    auto km_off = [](int kk) -> uint32_t { return (uint32_t)(((kk >> 2) * kHalf + (kk & 3) * 32) >> 4); };
    // MN-major operand, k-step kk: 16 rows of 128 bytes
    auto mn_off = [](int kk) -> uint32_t { return (uint32_t)((kk * 2048) >> 4); };
    auto issue_st = [&](int qs) {   // X = K Q^T
      const uint64_t bq = dQ_km + (uint64_t)(qs * (kTile >> 4));
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) umma_ss_w(tmem_base + X, dK_km + km_off(kk), bq + km_off(kk), idesc_kk, kk > 0 ? 1u : 0u, leader);
    };
    auto issue_dpt = [&]() {        // Y = V dO^T
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) umma_ss_w(tmem_base + Y, dV_km + km_off(kk), dDO_km + km_off(kk), idesc_kk, kk > 0 ? 1u : 0u, leader);
    };
    auto issue_dv = [&](bool accumulate) {   // dV += P^T dO; P^T of queries [32g, 32g+32) sits in X columns [32g, 32g+16)
#pragma unroll
      for (int kk = 0; kk < 8; ++kk)
        umma_ts_w(tmem_base + DV, tmem_base + X + (uint32_t)((kk >> 1) * 32 + (kk & 1) * 8), dDO_mn + mn_off(kk), idesc_kn,
                  (accumulate || kk > 0) ? 1u : 0u, leader);
    };
    auto issue_dq = [&]() {         // Y = K^T dS^T
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) umma_ss_w(tmem_base + Y, dK_mn + mn_off(kk), dDS_mn + mn_off(kk), idesc_mn, kk > 0 ? 1u : 0u, leader);
    };
    auto issue_dk = [&](int qs, bool accumulate) {   // dK += dS^T Q
      const uint64_t bq = dQ_mn + (uint64_t)(qs * (kTile >> 4));
#pragma unroll
      for (int kk = 0; kk < 8; ++kk)
        umma_ss_w(tmem_base + DK, dDS_km + km_off(kk), bq + mn_off(kk), idesc_kn, (accumulate || kk > 0) ? 1u : 0u, leader);
    };
    bool ok = wait_all(kv_full, 0);
    if (ok && n_q > 0) ok = wait_all(&q_full[0], 0);
    if (ok && n_q > 0) {
      tc_fence_after();
      issue_st(0);
      umma_commit_w(s_full, leader);
      ok = wait_all(do_full, 0);
    }
    if (ok && n_q > 0) {
      tc_fence_after();
      issue_dpt();
      umma_commit_w(dp_full, leader);
    }
    for (int i = 0; i < n_q && ok; ++i) {
      const uint32_t par = i & 1;
      const int qs = i % kQStages;
      const bool has_next = (i + 1) < n_q;
      if (!wait_all(p_ready, par)) { ok = false; break; }
      tc_fence_after();
      issue_dv(i > 0);
      umma_commit_w(do_empty, leader);          // dO(i) is free once dV(i) has completed
      if (has_next) {
        const int qn = (i + 1) % kQStages;
        if (!wait_all(&q_full[qn], ((i + 1) / kQStages) & 1)) { ok = false; break; }
        tc_fence_after();
        issue_st(qn);                           // executes after dV(i), which reads P^T out of X
        umma_commit_w(s_full, leader);
      }
      if (!wait_all(ds_ready, par)) { ok = false; break; }
      tc_fence_after();
      issue_dq();
      umma_commit_w(dq_full, leader);
      issue_dk(qs, i > 0);
      umma_commit_w(&q_empty[qs], leader);      // Q(i) is free once dK(i) has completed
      if (has_next) {
        if (!wait_all(dq_free, par)) { ok = false; break; }
        if (!wait_all(do_full, (i + 1) & 1)) { ok = false; break; }
        tc_fence_after();
        issue_dpt();
        umma_commit_w(dp_full, leader);
      }
    }
    if (ok && n_q > 0) umma_commit_w(done, leader);
    if (!ok && lane == 0) { atomicCAS(err, 0, 52); *abort_flag = 1; }
  } else if (warp >= kEwWarps) {
    // ------------------------------------------------------------------------------------------ dQ^T drain warps
    const int quarter = warp & 3;
    const int d = quarter * 32 + lane;                    // TMEM lane == head-dim index of dQ^T
    const uint32_t tY = tmem_base + Y + ((uint32_t)(quarter * 32) << 16);
    bool ok = true;
    for (int i = 0; i < n_q; ++i) {
      if (!mbar_wait(dq_full, i & 1, abort_flag)) { ok = false; break; }
      tc_fence_after();
#pragma unroll 1
      for (int half = 0; half < 2; ++half) {
        uint32_t a0[32], a1[32];
        tmem_ld32(tY + half * 64, a0);
        tmem_ld32(tY + half * 64 + 32, a1);
        tmem_ld_wait();
        if (half == 1) {                                   // Y may be overwritten by the next dP^T from here on
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(dq_free);
        }
        const int q0 = q_tile(i) * 128 + half * 64;
        // head-major accumulator [B, H, Sq, 128]: consecutive queries are 512 bytes apart, so every reduction below is one
        // instruction with an immediate offset from a single base pointer
        float* qrow = dQacc + (bh * Sq + (size_t)q0) * HD + d;
        if (q0 + 64 <= Sq) {
#pragma unroll
          for (int j = 0; j < 32; ++j) red_add_f32t(qrow + j * HD, __uint_as_float(a0[j]));
#pragma unroll
          for (int j = 0; j < 32; ++j) red_add_f32t(qrow + (32 + j) * HD, __uint_as_float(a1[j]));
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (q0 + j < Sq) red_add_f32t(qrow + j * HD, __uint_as_float(a0[j]));
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (q0 + 32 + j < Sq) red_add_f32t(qrow + (32 + j) * HD, __uint_as_float(a1[j]));
        }
      }
    }
    if (!ok && lane == 0) { atomicCAS(err, 0, 54); *abort_flag = 1; }
  } else {
    // ------------------------------------------------------------------------------------------ element-wise warps
    // warp = cg * 4 + quarter: TMEM lanes [32 quarter, +32) (key rows), query columns [32 cg, +32)
    const int quarter = warp & 3, cg = warp >> 2;
    const int row = quarter * 32 + lane;            // key row inside the tile == TMEM lane
    const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
    const uint32_t tX = tmem_base + X + lane_off + cg * 32;
    const uint32_t tY = tmem_base + Y + lane_off + cg * 32;
    // dS^T tile: half (cg >> 1) holds queries [64 (cg>>1), +64); inside it this thread's 32 queries are 16-byte chunks
    // (cg & 1) * 4 .. + 3 of row `row`, XOR-swizzled with the row index
    uint8_t* ds_row = sDS + (cg >> 1) * kHalf + row * 128;
    const int sw = row & 7, chunk0 = (cg & 1) * 4;
    const float2 sc2 = make_float2(scale_log2, scale_log2);
    // NA: this thread's key coordinates (tile blockIdx.x, row dt * 32 + dh * 8 + dw)
    int k_t = 0, k_h = 0, k_w = 0;
    if (NA) {
      const int kt = blockIdx.x;
      k_t = (kt / (na.nH * na.nW)) * 4 + (row >> 5);
      k_h = ((kt / na.nW) % na.nH) * 4 + ((row >> 3) & 3);
      k_w = (kt % na.nW) * 8 + (row & 7);
    }
    bool ok = true;
    for (int i = 0; i < n_q; ++i) {
      const uint32_t par = i & 1;
      const int ss = i & 1;
      // visibility of this thread's 32 queries (dt = cg, bit dh * 8 + dw): all ones for a fully visible tile pair
      uint32_t vis = 0xffffffffu;
      if (NA) {
        const int entry = my_list[i];
        if (entry >= 0) {
          const int qt = entry;
          const uint32_t mt = na.bt[k_t * na.nT + qt / (na.nH * na.nW)];
          const uint32_t mh = na.bh[k_h * na.nH + (qt / na.nW) % na.nH];
          const uint32_t mw = na.bw[k_w * na.nW + qt % na.nW];
          vis = 0u;
          if ((mt >> cg) & 1u) {
#pragma unroll
            for (int dh = 0; dh < 4; ++dh) vis |= ((mh >> dh) & 1u) ? (mw << (dh * 8)) : 0u;
          }
        }
      }
      if (!mbar_wait(&st_full[ss], (i >> 1) & 1, abort_flag)) { ok = false; break; }
      if (!mbar_wait(s_full, par, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const float4* l4 = reinterpret_cast<const float4*>(sStat + ss * 256 + cg * 32);   // -lse * log2(e)
      const float4* d4 = l4 + 32;                                                       // -delta
      // ---- phase 1: P^T = exp2(S^T * c - lse); the fp32 values stay in registers for phase 2
      uint32_t p[32];
      tmem_ld32(tX, p);
      tmem_ld_wait();
      {
        uint32_t pp[16];
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          const float4 nl = l4[g];
          const float2 x0 = fma2(make_float2(__uint_as_float(p[g * 4]), __uint_as_float(p[g * 4 + 1])), sc2, make_float2(nl.x, nl.y));
          const float2 x1 = fma2(make_float2(__uint_as_float(p[g * 4 + 2]), __uint_as_float(p[g * 4 + 3])), sc2, make_float2(nl.z, nl.w));
          float e0 = ex2t(x0.x), e1 = ex2t(x0.y), e2 = ex2t(x1.x), e3 = ex2t(x1.y);
          if (NA && vis != 0xffffffffu) {
            e0 = ((vis >> (g * 4)) & 1u) ? e0 : 0.f;
            e1 = ((vis >> (g * 4 + 1)) & 1u) ? e1 : 0.f;
            e2 = ((vis >> (g * 4 + 2)) & 1u) ? e2 : 0.f;
            e3 = ((vis >> (g * 4 + 3)) & 1u) ? e3 : 0.f;
          }
          p[g * 4] = __float_as_uint(e0);
          p[g * 4 + 1] = __float_as_uint(e1);
          p[g * 4 + 2] = __float_as_uint(e2);
          p[g * 4 + 3] = __float_as_uint(e3);
          __nv_bfloat162 a0 = __floats2bfloat162_rn(e0, e1), a1 = __floats2bfloat162_rn(e2, e3);
          pp[g * 2] = *reinterpret_cast<uint32_t*>(&a0);
          pp[g * 2 + 1] = *reinterpret_cast<uint32_t*>(&a1);
        }
        // bf16 P^T of these 32 queries goes over the first 16 of the 32 columns this warp has just read: no other warp's data
        tmem_st16(tX, pp);
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_ready);

      // ---- phase 2: dS^T = P^T o (dP^T - delta) -> shared memory
      if (!mbar_wait(dp_full, par, abort_flag)) { ok = false; break; }
      tc_fence_after();
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        uint32_t dp[16];
        tmem_ld16(tY + hh * 16, dp);
        tmem_ld_wait();
        uint32_t pd[8];
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          const float4 nd = d4[hh * 4 + g];
          const int e = hh * 16 + g * 4;
          const float2 t0 = add2(make_float2(__uint_as_float(dp[g * 4]), __uint_as_float(dp[g * 4 + 1])), make_float2(nd.x, nd.y));
          const float2 t1 = add2(make_float2(__uint_as_float(dp[g * 4 + 2]), __uint_as_float(dp[g * 4 + 3])), make_float2(nd.z, nd.w));
          const float2 s0 = mul2(make_float2(__uint_as_float(p[e]), __uint_as_float(p[e + 1])), t0);
          const float2 s1 = mul2(make_float2(__uint_as_float(p[e + 2]), __uint_as_float(p[e + 3])), t1);
          __nv_bfloat162 b0 = __floats2bfloat162_rn(s0.x, s0.y), b1 = __floats2bfloat162_rn(s1.x, s1.y);
          pd[g * 2] = *reinterpret_cast<uint32_t*>(&b0);
          pd[g * 2 + 1] = *reinterpret_cast<uint32_t*>(&b1);
        }
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const uint4 v = make_uint4(pd[j * 4], pd[j * 4 + 1], pd[j * 4 + 2], pd[j * 4 + 3]);
          *reinterpret_cast<uint4*>(ds_row + (((chunk0 + hh * 2 + j) ^ sw) << 4)) = v;
        }
      }
      fence_proxy_async();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(ds_ready);
        mbar_arrive(&st_empty[ss]);
      }
    }
    if (ok && n_q > 0) ok = mbar_wait(done, 0, abort_flag);
    if (ok) {
      tc_fence_after();
      // warps with cg 0,1 write dV, cg 2,3 write dK (scaled); the two warps of a lane quarter take 64 columns each
      const int which = cg >> 1, half = cg & 1;
      const int kv_row = kv_base + row;
      const uint32_t tAcc = tmem_base + (which == 0 ? DV : DK) + lane_off;
      const float mul = (which == 0) ? 1.f : scale;
      bf16* base = (which == 0) ? dV : dK;
      bf16* orow = base + (((size_t)b * Skv + (kv_row < Skv ? kv_row : 0)) * H + h) * HD;
#pragma unroll 1
      for (int c = half * 2; c < half * 2 + 2; ++c) {
        uint32_t o[32];
        tmem_ld32(tAcc + c * 32, o);
        tmem_ld_wait();
        if (n_q == 0) {               // no query sees this key tile: its gradients are zero (the accumulators were never written)
#pragma unroll
          for (int j = 0; j < 32; ++j) o[j] = 0u;
        }
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

// Runs after the preprocessing kernel has produced lse2 / delta (negated, padded to S_pad rows per (b, h); S_pad a multiple of 128).
// dq_acc: B*Sq*H*128 floats of scratch, zeroed here; converted to bf16 dq (times `scale`) by the caller's convert kernel.
extern "C" int cb200_fa_bwd_tile_main(const void* d_o, const void* q, const void* k, const void* v, const float* lse2,
                                      const float* delta, float* dq_acc, void* dk, void* dv, int B, int Sq, int Skv, int H, int S_pad,
                                      float scale, int* err, cudaStream_t st) {
  using namespace fat;
  if (S_pad % 128 != 0) return -41;
  auto make = [&](CUtensorMap* m, const void* p, int S) {
    const uint64_t dims[4] = {(uint64_t)HD, (uint64_t)H, (uint64_t)S, (uint64_t)B};
    const uint64_t strides[3] = {(uint64_t)HD * 2, (uint64_t)H * HD * 2, (uint64_t)S * H * HD * 2};
    const uint32_t box[4] = {64, 1, 128, 1};
    return make_tmap_bf16(m, p, 4, dims, strides, box);
  };
  CUtensorMap tq, tdo, tk, tv;
  int rc = make(&tq, q, Sq) | make(&tdo, d_o, Sq) | make(&tk, k, Skv) | make(&tv, v, Skv);
  if (rc) return rc;
  static bool attr = false;
  if (!attr) {
    cudaError_t e = cudaFuncSetAttribute(fa_bwd_tile_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmem);
    if (e != cudaSuccess) return 300 + (int)e;
    attr = true;
  }
  const size_t n = (size_t)B * Sq * H * HD;
  cudaError_t e = cudaMemsetAsync(dq_acc, 0, n * sizeof(float), st);
  if (e != cudaSuccess) return 400 + (int)e;
  dim3 grid((Skv + 127) / 128, H, B);
  fa_bwd_tile_kernel<false><<<grid, kThreads, kSmem, st>>>(tq, tdo, tk, tv, lse2, delta, dq_acc, (bf16*)dk, (bf16*)dv, Sq, Skv, H, S_pad,
                                                           scale, NaBwdPlan{}, err);
  return (int)cudaGetLastError();
}

// Neighbourhood attention backward. q, k, v, d_o and the outputs are in tile order ([B, S, H, 128] with S = nT * nH * nW tiles of 128
// rows, row dt * 32 + dh * 8 + dw inside a tile); lse2 / delta as above, in the same order. q_list [S / 128][max_n] int32 (top bit:
// whole tile pair visible), q_cnt [S / 128]; bt / bh / bw: uint8 tables [4 nT][nT], [4 nH][nH], [8 nW][nW].
extern "C" int cb200_fa_bwd_tile_na(const void* d_o, const void* q, const void* k, const void* v, const float* lse2, const float* delta,
                                    float* dq_acc, void* dk, void* dv, int B, int S, int H, float scale, const int* q_list,
                                    const int* q_cnt, int max_n, const uint8_t* bt, const uint8_t* bh, const uint8_t* bw, int nT, int nH,
                                    int nW, int* err, cudaStream_t st) {
  using namespace fat;
  if (S != nT * nH * nW * 128 || max_n < 1) return -42;
  auto make = [&](CUtensorMap* m, const void* p) {
    const uint64_t dims[4] = {(uint64_t)HD, (uint64_t)H, (uint64_t)S, (uint64_t)B};
    const uint64_t strides[3] = {(uint64_t)HD * 2, (uint64_t)H * HD * 2, (uint64_t)S * H * HD * 2};
    const uint32_t box[4] = {64, 1, 128, 1};
    return make_tmap_bf16(m, p, 4, dims, strides, box);
  };
  CUtensorMap tq, tdo, tk, tv;
  int rc = make(&tq, q) | make(&tdo, d_o) | make(&tk, k) | make(&tv, v);
  if (rc) return rc;
  static bool attr = false;
  if (!attr) {
    cudaError_t e = cudaFuncSetAttribute(fa_bwd_tile_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmem);
    if (e != cudaSuccess) return 300 + (int)e;
    attr = true;
  }
  cudaError_t e = cudaMemsetAsync(dq_acc, 0, (size_t)B * S * H * HD * sizeof(float), st);
  if (e != cudaSuccess) return 400 + (int)e;
  dim3 grid(S / 128, H, B);
  fa_bwd_tile_kernel<true><<<grid, kThreads, kSmem, st>>>(tq, tdo, tk, tv, lse2, delta, dq_acc, (bf16*)dk, (bf16*)dv, S, S, H, S, scale,
                                                          NaBwdPlan{q_list, q_cnt, bt, bh, bw, max_n, nT, nH, nW}, err);
  return (int)cudaGetLastError();
}
