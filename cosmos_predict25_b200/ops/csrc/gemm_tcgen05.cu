// bf16 GEMM on the 5th-generation tensor cores (sm_100a): C[M,N] = epilogue(A x B), fp32 accumulation.
//
// Persistent, warp-specialised kernel, one CTA per SM:
//   warp 0   TMA producer: streams 128x64 A tiles and 256x64 B tiles (128-byte swizzle) through a
//            4-stage shared-memory ring; completion by mbarrier transaction bytes.
//   warp 1   MMA issuer: one thread issues tcgen05.mma (UMMA 128x256x16, cta_group::1) from
//            shared-memory descriptors into one of two 128x256 fp32 accumulators in TMEM
//            (2 x 256 = all 512 columns), and releases ring slots with tcgen05.commit.
//   warps 2-5 epilogue: tcgen05.ld the finished accumulator (each warp owns one 32-lane quarter of
//            TMEM), apply the fused epilogue in registers and store bf16 straight to global memory,
//            while warp 1 already accumulates the next tile into the other TMEM buffer.
//
// Operand majors are template parameters so the same kernel serves forward (x @ W^T: both K-major),
// dgrad (dy @ W: B is N-major) and wgrad (dy^T @ x: both MN-major) without transposing in memory.
// Fused epilogues: + bias, exact GELU (optionally also writing the pre-activation for backward),
// and the AdaLN gated residual  out = resid + gate[row / L, col] * acc.
//
// FSDP all-gather fused into the GEMM (template flag GATHER): the B operand is a weight [rows, ld] whose rows are sharded over P
// ranks (rank r holds rows [r * chunk_rows, (r + 1) * chunk_rows) in its own memory). Four extra warps per CTA pull the shards -
// plain 16-byte loads from the owners' memory, local or over NVLink - into a local full-size copy, in groups of 256 rows cut into
// slices, and publish every finished slice with a release increment of the group's counter. The TMA producer acquires the
// counter of the group a B box lies in before it issues the load, so tiles are computed while later groups are still in
// flight and every remote row crosses NVLink exactly once. The same code serves the forward GEMM (groups along N) and dgrad
// (groups along the contraction dimension).
//
// All mbarrier waits are bounded; on timeout the CTA records an error code in `err`, lets in-flight
// copies land, frees its TMEM and returns.

#include <math.h>

#include "launchers.h"
#include <algorithm>
#include <cstdlib>

#include "common.cuh"
#include "sm100.cuh"
#include "tmap.h"

namespace cb200 {
using namespace sm100;

constexpr int BM = 128, BN = 256, BK = 64, UK = 16;
constexpr int kStages = 4;
constexpr int kABytes = BM * BK * 2;  // 16 KB
constexpr int kBBytes = BN * BK * 2;  // 32 KB
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kGemmThreads = 320;  // TMA warp, MMA warp, 8 epilogue warps (two per TMEM lane quarter, 128 columns each)
constexpr int kStageOutBytes = 8 * 32 * 128;  // one 32-row x 128-byte staging block per epilogue warp
constexpr size_t kSmemBytes = (size_t)kStages * kStageBytes + 1024 /*alignment slack*/ + 256 /*barriers*/ + kStageOutBytes;

// Ulysses exchange fused into the epilogue: the output [M, N] is a projection to H = N / 128 heads of a local sequence of S
// tokens per batch item; head h of token (b, s) is normalised (optional per-head RMSNorm), rotated (optional rotate-half
// RoPE) and stored straight into the staging buffer of the rank that owns the head, at its place in the gathered sequence.
struct HeadScatter {
  int64_t ptrs[8];    // staging buffers of the P ranks, each [B, P * S, Hl, 128] bf16
  const float* w;     // [128] RMSNorm weight or nullptr
  const float* cosv;  // [S, 64] or nullptr
  const float* sinv;
  int S, Hl, P, rank;
  float eps;
  bf16* raw;          // optional [M, N]: the un-normalised projection, kept locally for the RMSNorm backward (training)
  float* rstd_out;    // optional [M, N / 128]: reciprocal RMS of every (token, head), with ``raw``
};

struct GemmEpilogue {
  HeadScatter hs;     // hs.P == 0: disabled
  bf16* C;
  bf16* pre;          // optional second output: the pre-activation (act == 1) or the product before the gated residual
                      // (full 256-column tiles only)
  const bf16* bias;   // optional [N]
  const bf16* resid;  // optional [M, N] (gated residual)
  const float* gate;  // optional [M / L, N]
  int act;            // 0 none, 1 gelu(erf)
  int L;              // rows per gate vector
};

__device__ __forceinline__ float gelu_erf(float x) { return 0.5f * x * (1.f + erff(x * 0.70710678118654752f)); }

// Row-sharded B operand gathered inside the kernel (see the header comment).
constexpr int kGatherWarps = 2;   // with the 10 GEMM warps: three warpgroups, 168 registers per thread (four more warps
                                  // would cap the epilogue at 128 registers and make it spill)
constexpr int kGatherGroupRows = 256;
struct GatherB {
  int64_t ptrs[8];     // rank r: its rows [r * chunk_rows, ...) of the weight, row-major with `ld` elements per row
  bf16* ws;            // local full copy [rows, ld]; the B tensor map is built on it
  int* counters;       // one per 256-row group, zeroed by the host before the launch
  int P, chunk_rows, rows, ld;
  int slices;          // pieces a group is cut into; a group is complete when its counter reaches this value
};

__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_gpu_add(int* p, int v) {
  asm volatile("red.release.gpu.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// CTA2: two CTAs of a cluster share one 256 x 256 output tile (tcgen05 cta_group::2). CTA r of the pair loads rows
// [128 r, 128 r + 128) of the A tile and of the B tile into its own shared memory (half the B bytes per CTA and per MMA), the even
// CTA issues M = 256 MMAs that read both shared memories, each CTA's TMEM receives its 128 rows and its epilogue warps drain them.
// Six 32 KB stages instead of four 48 KB ones.
template <int A_MN, int B_MN, bool GATHER, bool CTA2 = false>
__global__ void __launch_bounds__(kGemmThreads + (GATHER ? kGatherWarps * 32 : 0), 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b, int M, int N, int K,
                 GemmEpilogue ep, GatherB gb, int* __restrict__ err) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  static_assert(!(CTA2 && GATHER), "the gather mode runs on single-CTA tiles");
  constexpr int STG = CTA2 ? 6 : kStages;                                   // pipeline stages
  constexpr int STG_BYTES = CTA2 ? (kABytes + kBBytes / 2) : kStageBytes;   // bytes per stage in this CTA
  constexpr int TM = CTA2 ? 2 * BM : BM;                                    // output rows per tile (per pair with CTA2)
  static_assert(STG * STG_BYTES == kStages * kStageBytes, "both layouts fill the same shared-memory window");
  const uint32_t pair_rank = CTA2 ? cluster_ctarank() : 0u;
  const int first_tile = CTA2 ? (int)(blockIdx.x >> 1) : (int)blockIdx.x, tile_step = CTA2 ? (int)(gridDim.x >> 1) : (int)gridDim.x;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STG * STG_BYTES);
  uint64_t* full = bars;                    // [STG]
  uint64_t* empty = bars + STG;             // [STG]
  uint64_t* acc_full = bars + 2 * STG;      // [2]
  uint64_t* acc_empty = acc_full + 2;       // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  // the shuffle makes the warp index (and every role branch below) provably warp-uniform for the compiler
  const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;
  const int tiles_m = (M + TM - 1) / TM, tiles_n = (N + BN - 1) / BN;
  const int n_tiles = tiles_m * tiles_n;
  const int k_blocks = (K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STG; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], CTA2 ? 16 : 8);      // the pair leader hears from the epilogue warps of both CTAs
    }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    if (CTA2) {
      tmem_alloc_pair(tmem_slot, 512);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(tmem_slot, 512);
      tmem_relinquish();
    }
  }
  tc_fence_before();
  __syncthreads();
  if (CTA2) cluster_sync_all();      // the other CTA's barriers exist before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      prefetch_tmap(&tma_a);
      prefetch_tmap(&tma_b);
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      // GATHER: groups of B rows whose gather this thread has already seen complete (a bit per group, 128 groups)
      unsigned long long seen[2] = {0ull, 0ull};
      auto group_ready = [&](int row) -> bool {
        const int g = row / kGatherGroupRows;
        if (g < 128 && ((seen[g >> 6] >> (g & 63)) & 1ull)) return true;
        const unsigned long long t0 = global_timer_ns();
        while (ld_acquire_gpu(gb.counters + g) < gb.slices) {
          __nanosleep(64);
          if (*abort_flag || global_timer_ns() - t0 > kWaitLimitNs) return false;
        }
        fence_proxy_async_all();    // the rows were written by ordinary stores; the TMA load below reads them through the async proxy
        if (g < 128) seen[g >> 6] |= 1ull << (g & 63);
        return true;
      };
      for (int t = first_tile; t < n_tiles && ok; t += tile_step) {
        // with CTA2 this CTA fetches its 128 rows of the pair's A tile and its 128 rows of the B tile
        const int m0 = (t / tiles_n) * TM + (CTA2 ? (int)pair_rank * BM : 0), n0 = (t % tiles_n) * BN + (CTA2 ? (int)pair_rank * (BN / 2) : 0);
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (GATHER) {
            // rows of the weight this stage reads: an N tile of 256 rows (forward) or 64 rows of the contraction dimension (dgrad)
            if (B_MN == 0) {
              if (kb == 0 && !group_ready(n0)) { ok = false; break; }
            } else if (!group_ready(kb * BK)) { ok = false; break; }
          }
          if (!mbar_wait(&empty[s], ph ^ 1, abort_flag)) { ok = false; break; }
          uint8_t* sa = smem + s * STG_BYTES;
          uint8_t* sb = sa + kABytes;
          const int k0 = kb * BK;
          if (CTA2) {
            // all bytes of the pair's stage are counted on the leader's barrier: the leader announces them, both CTAs load
            if (pair_rank == 0) mbar_arrive_expect_tx(&full[s], 2 * STG_BYTES);
            const uint32_t bar = mapa_shared(smem_u32(&full[s]), 0);
            if (A_MN == 0) {
              tma_load_2d_pair(sa, &tma_a, bar, k0, m0);
            } else {
#pragma unroll
              for (int j = 0; j < BM / 64; ++j) tma_load_2d_pair(sa + j * 8192, &tma_a, bar, m0 + j * 64, k0);
            }
            if (B_MN == 0) {
              tma_load_2d_pair(sb, &tma_b, bar, k0, n0);
            } else {
#pragma unroll
              for (int j = 0; j < BN / 128; ++j) tma_load_2d_pair(sb + j * 8192, &tma_b, bar, n0 + j * 64, k0);
            }
          } else {
            mbar_arrive_expect_tx(&full[s], kStageBytes);
            if (A_MN == 0) {
              tma_load_2d(sa, &tma_a, &full[s], k0, m0);
            } else {
#pragma unroll
              for (int j = 0; j < BM / 64; ++j) tma_load_2d(sa + j * 8192, &tma_a, &full[s], m0 + j * 64, k0);
            }
            if (B_MN == 0) {
              tma_load_2d(sb, &tma_b, &full[s], k0, n0);
            } else {
#pragma unroll
              for (int j = 0; j < BN / 64; ++j) tma_load_2d(sb + j * 8192, &tma_b, &full[s], n0 + j * 64, k0);
            }
          }
          if (++s == STG) { s = 0; ph ^= 1; }
        }
      }
      if (!ok) { atomicCAS(err, 0, 1); *abort_flag = 1; }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    // The whole warp runs this loop with identical values and only the elected lane issues: warp-uniform control flow and
    // descriptor arithmetic stay on the uniform datapath, which lowers the issue cost per MMA.
    {
      const uint32_t leader = elect_one() ? 1u : 0u;
      auto wait_all = [&](uint64_t* bar, uint32_t parity) -> bool { return __all_sync(0xffffffffu, mbar_wait(bar, parity, abort_flag)); };
      constexpr uint32_t idesc = umma_idesc_bf16(TM, BN, A_MN, B_MN);
      // stage-0 descriptors; a stage / k-slice is a constant added to the address field (16-byte units)
      const uint64_t da0 = A_MN ? umma_desc_sw128(smem_u32(smem), 8192, 1024) : umma_desc_sw128(smem_u32(smem), 16, 1024);
      const uint64_t db0 = B_MN ? umma_desc_sw128(smem_u32(smem) + kABytes, 8192, 1024) : umma_desc_sw128(smem_u32(smem) + kABytes, 16, 1024);
      int s = 0;
      uint32_t ph = 0;
      int acc = 0;
      uint32_t acc_ph = 0;
      bool ok = true;
      for (int t = first_tile; t < n_tiles && ok && pair_rank == 0; t += tile_step) {     // only the pair leader issues
        if (!wait_all(&acc_empty[acc], acc_ph ^ 1)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!wait_all(&full[s], ph)) { ok = false; break; }
          tc_fence_after();
          const uint64_t da_s = da0 + (uint64_t)(s * (STG_BYTES >> 4)), db_s = db0 + (uint64_t)(s * (STG_BYTES >> 4));
#pragma unroll
          for (int k = 0; k < BK / UK; ++k) {
            const uint64_t da = da_s + (uint32_t)((A_MN ? k * (UK * 128) : k * (UK * 2)) >> 4);
            const uint64_t db = db_s + (uint32_t)((B_MN ? k * (UK * 128) : k * (UK * 2)) >> 4);
            if (CTA2) umma_ss_pair_w(d_tmem, da, db, idesc, (kb > 0 || k > 0) ? 1u : 0u, leader);
            else umma_ss_w(d_tmem, da, db, idesc, (kb > 0 || k > 0) ? 1u : 0u, leader);
          }
          // slot reusable once these MMAs have read it (with CTA2: in both CTAs)
          if (CTA2) umma_commit_pair_w(&empty[s], leader);
          else umma_commit_w(&empty[s], leader);
          if (++s == STG) { s = 0; ph ^= 1; }
        }
        if (!ok) break;
        if (CTA2) umma_commit_pair_w(&acc_full[acc], leader);
        else umma_commit_w(&acc_full[acc], leader);
        if (++acc == 2) { acc = 0; acc_ph ^= 1; }
      }
      if (!ok && lane == 0) { atomicCAS(err, 0, 2); *abort_flag = 1; }
    }
  } else if (GATHER && warp >= 10) {
    // ------------------------------------------------------------------ gather warps
    // item = (group, slice); CTA b takes items b, b + grid, ...; item i works on group i % n_groups, so the CTAs' first
    // items cover every group at once and the group of a CTA's own first tile is among the first to complete
    const int tid = threadIdx.x - 10 * 32;
    const int n_groups = (gb.rows + kGatherGroupRows - 1) / kGatherGroupRows;
    const int n_items = n_groups * gb.slices;
    const int row_vecs = gb.ld >> 3;                       // 16-byte pieces per row
    for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
      const int g = item % n_groups, sl = item / n_groups;
      const int g_lo = g * kGatherGroupRows, g_hi = min(gb.rows, g_lo + kGatherGroupRows);
      const int per = (g_hi - g_lo + gb.slices - 1) / gb.slices;
      const int r_lo = min(g_hi, g_lo + sl * per), r_hi = min(g_hi, r_lo + per);
      const long n_vec = (long)(r_hi - r_lo) * row_vecs;
      // 16 independent 16-byte loads per thread and round: enough bytes in flight per SM to cover the NVLink round trip
      constexpr int kInFlight = 16;
      // consecutive lanes take consecutive 16-byte pieces: one warp load is 512 contiguous bytes on the link
      constexpr int kGatherThreads = kGatherWarps * 32;
      for (long v0 = tid; v0 < n_vec; v0 += (long)kGatherThreads * kInFlight) {
        uint4 buf[kInFlight];
#pragma unroll
        for (int u = 0; u < kInFlight; ++u) {
          const long v = v0 + (long)u * kGatherThreads;
          if (v < n_vec) {
            const int row = r_lo + (int)(v / row_vecs), piece = (int)(v % row_vecs);
            const int owner = row / gb.chunk_rows;
            const bf16* src = reinterpret_cast<const bf16*>(gb.ptrs[owner]) + (size_t)(row - owner * gb.chunk_rows) * gb.ld;
            buf[u] = *(reinterpret_cast<const uint4*>(src) + piece);
          }
        }
#pragma unroll
        for (int u = 0; u < kInFlight; ++u) {
          const long v = v0 + (long)u * kGatherThreads;
          if (v < n_vec) {
            const int row = r_lo + (int)(v / row_vecs), piece = (int)(v % row_vecs);
            *(reinterpret_cast<uint4*>(gb.ws + (size_t)row * gb.ld) + piece) = buf[u];
          }
        }
      }
      __threadfence();
      asm volatile("bar.sync 1, %0;" ::"n"(kGatherWarps * 32) : "memory");   // every gather thread has stored and fenced
      if (tid == 0) red_release_gpu_add(gb.counters + g, 1);
    }
  } else {
    // ------------------------------------------------------------------ epilogue warps
    const int quarter = warp & 3;      // TMEM lanes [32*quarter, 32*quarter + 32)
    const int part = (warp - 2) >> 2;  // accumulator columns [128*part, 128*part + 128)
    uint8_t* stage_warp = smem + STG * STG_BYTES + 256 + (warp - 2) * (32 * 128);
    uint8_t* stage_row = stage_warp + lane * 128;
    int acc = 0;
    uint32_t acc_ph = 0;
    bool ok = true;
    const bool vec_ok = (N % 8) == 0;
    const uint32_t acc_empty_leader[2] = {CTA2 ? mapa_shared(smem_u32(&acc_empty[0]), 0) : 0u,
                                          CTA2 ? mapa_shared(smem_u32(&acc_empty[1]), 0) : 0u};
    for (int t = first_tile; t < n_tiles && ok; t += tile_step) {
      const int m0 = (t / tiles_n) * TM + (CTA2 ? (int)pair_rank * BM : 0), n0 = (t % tiles_n) * BN;
      if (!mbar_wait(&acc_full[acc], acc_ph, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const int row = m0 + quarter * 32 + lane;
      const uint32_t t_row = tmem_base + acc * BN + ((uint32_t)(quarter * 32) << 16);
      if (ep.hs.P > 0) {
        // ---- fused head scatter: this thread owns one token row; a 256-wide tile holds two complete heads
        // tcgen05.ld is warp-collective: every lane runs every load, rows past M only skip their stores
        const bool valid = row < M;
        {
          const int row_c = valid ? row : M - 1;
          const int b_idx = row_c / ep.hs.S, s_idx = row_c % ep.hs.S;
          for (int hh = part; hh == part; ++hh) {      // this warp's head of the tile
            const int head = (n0 + hh * 128) >> 7;
            if ((head + 1) * 128 > N) break;
            const uint32_t t_head = t_row + hh * 128;
            float rstd = 1.f;
            if (ep.hs.w != nullptr) {          // pass 1: sum of squares over the head (TMEM re-reads are cheap)
              float ss = 0.f;
#pragma unroll 1
              for (int c = 0; c < 4; ++c) {
                uint32_t r[32];
                tmem_ld32(t_head + c * 32, r);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 32; ++j) ss = fmaf(__uint_as_float(r[j]), __uint_as_float(r[j]), ss);
              }
              rstd = rsqrtf(ss * (1.f / 128.f) + ep.hs.eps);
              if (ep.hs.rstd_out != nullptr && valid) ep.hs.rstd_out[(size_t)row * (N >> 7) + head] = rstd;
            }
            const unsigned long long raw_u =
                ep.hs.raw != nullptr ? reinterpret_cast<unsigned long long>(ep.hs.raw + (size_t)row_c * N + (size_t)head * 128) : 0ull;
            const int dst_rank = head / ep.hs.Hl, hl = head - dst_rank * ep.hs.Hl;
            bf16* dst = reinterpret_cast<bf16*>(ep.hs.ptrs[dst_rank]) +
                        ((((size_t)b_idx * ep.hs.P + ep.hs.rank) * ep.hs.S + s_idx) * ep.hs.Hl + hl) * 128;
            int c_cur = 0;
            // this thread's row (columns [32c, 32c + 32) in ``lo32`` and their rotation partners [64 + 32c, ...) in ``hi32``) goes to
            // the warp's staging block, 16-byte chunks XOR-swizzled by the row (no bank conflicts); then 4 lanes cover a 64-byte
            // run of a head row, so a warp store is eight contiguous 64-byte segments (local memory or a peer's over NVLink)
            // instead of 32 scattered 16-byte pieces
            auto emit = [&](const float (&lo32)[32], const float (&hi32)[32], unsigned long long dst_u) {
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                uint4 o0, o1;
                __nv_bfloat162* p0 = reinterpret_cast<__nv_bfloat162*>(&o0);
                __nv_bfloat162* p1 = reinterpret_cast<__nv_bfloat162*>(&o1);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  p0[j] = __floats2bfloat162_rn(lo32[q * 8 + 2 * j], lo32[q * 8 + 2 * j + 1]);
                  p1[j] = __floats2bfloat162_rn(hi32[q * 8 + 2 * j], hi32[q * 8 + 2 * j + 1]);
                }
                *reinterpret_cast<uint4*>(stage_row + ((q ^ (lane & 7)) << 4)) = o0;
                *reinterpret_cast<uint4*>(stage_row + (((4 + q) ^ (lane & 7)) << 4)) = o1;
              }
              __syncwarp();
#pragma unroll 4
              for (int it = 0; it < 8; ++it) {
                const int r_src = it * 4 + (lane >> 3), chunk = lane & 7;
                const unsigned long long d = __shfl_sync(0xffffffffu, dst_u, r_src);
                const int ok_row = __shfl_sync(0xffffffffu, (int)valid, r_src);
                const uint4 v = *reinterpret_cast<const uint4*>(stage_warp + r_src * 128 + ((chunk ^ (r_src & 7)) << 4));
                const int col = (chunk < 4 ? c_cur * 32 + chunk * 8 : 64 + c_cur * 32 + (chunk - 4) * 8);
                if (ok_row) *reinterpret_cast<uint4*>(d + col * 2) = v;
              }
              __syncwarp();
            };
#pragma unroll 1
            for (int c = 0; c < 2; ++c) {      // pass 2: columns [32c, 32c+32) and their rotation partners [64+32c, 64+32c+32)
              uint32_t lo[32], hi[32];
              tmem_ld32(t_head + c * 32, lo);
              tmem_ld32(t_head + 64 + c * 32, hi);
              tmem_ld_wait();
              float a[32], bb[32];
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                a[j] = __uint_as_float(lo[j]);
                bb[j] = __uint_as_float(hi[j]);
              }
              c_cur = c;
              if (raw_u != 0ull) emit(a, bb, raw_u);        // warp-uniform: every lane of the kernel sees the same ep.hs.raw
              if (ep.hs.w != nullptr) {
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                  a[j] *= rstd * ep.hs.w[c * 32 + j];
                  bb[j] *= rstd * ep.hs.w[64 + c * 32 + j];
                }
                if (ep.hs.cosv != nullptr) {
                  // this row's 32 cosines and sines come in through the staging block with coalesced loads (8 lanes per
                  // 128-byte run, 4 rows per instruction); reading them per thread straight from global memory would be
                  // 32 scattered 16-byte loads per instruction
                  float cs[32], sn[32];
                  auto fetch_rows = [&](const float* table, float (&out)[32]) {
#pragma unroll 4
                    for (int it = 0; it < 8; ++it) {
                      const int r_src = it * 4 + (lane >> 3), chunk = lane & 7;
                      const int s_src = __shfl_sync(0xffffffffu, s_idx, r_src);
                      const uint4 v4 = *reinterpret_cast<const uint4*>(table + (size_t)s_src * 64 + c * 32 + chunk * 4);
                      *reinterpret_cast<uint4*>(stage_warp + r_src * 128 + ((chunk ^ (r_src & 7)) << 4)) = v4;
                    }
                    __syncwarp();
#pragma unroll
                    for (int q = 0; q < 8; ++q) {
                      const float4 f = *reinterpret_cast<const float4*>(stage_row + ((q ^ (lane & 7)) << 4));
                      out[q * 4] = f.x; out[q * 4 + 1] = f.y; out[q * 4 + 2] = f.z; out[q * 4 + 3] = f.w;
                    }
                    __syncwarp();
                  };
                  fetch_rows(ep.hs.cosv, cs);
                  fetch_rows(ep.hs.sinv, sn);
#pragma unroll
                  for (int j = 0; j < 32; ++j) {
                    const float x0 = a[j], x1 = bb[j], cc = cs[j], s1 = sn[j];
                    a[j] = x0 * cc - x1 * s1;
                    bb[j] = x1 * cc + x0 * s1;
                  }
                }
              }
              emit(a, bb, reinterpret_cast<unsigned long long>(dst));
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          if (CTA2) mbar_arrive_cluster(acc_empty_leader[acc]);
          else mbar_arrive(&acc_empty[acc]);
        }
        if (++acc == 2) { acc = 0; acc_ph ^= 1; }
        continue;
      }
      const float* gate_row = (ep.gate != nullptr && row < M) ? ep.gate + (size_t)(row / ep.L) * N : nullptr;
      if (vec_ok && n0 + BN <= N) {
        // ---- full-width tile: every global access of the epilogue goes through the warp's 4 KB staging block, so that a
        // warp instruction moves four contiguous 128-byte row segments instead of 32 scattered 16-byte pieces (the scattered
        // form made K = 2048 GEMMs epilogue-bound).  This warp owns 128 columns: two passes of 64; TMEM loads stay
        // warp-uniform.
        const int row0 = m0 + quarter * 32;
        auto write_out = [&](bf16* base, int colbase) {       // staged [32 rows x 64 cols] -> base[row, colbase ...]
          __syncwarp();
#pragma unroll 4
          for (int it = 0; it < 8; ++it) {
            const int r_src = it * 4 + (lane >> 3), chunk = lane & 7;
            const uint4 v4 = *reinterpret_cast<const uint4*>(stage_warp + r_src * 128 + ((chunk ^ (r_src & 7)) << 4));
            if (row0 + r_src < M) *reinterpret_cast<uint4*>(base + (size_t)(row0 + r_src) * N + colbase + chunk * 8) = v4;
          }
          __syncwarp();
        };
        auto stage_chunk = [&](int c, const float (&v)[32]) {   // this thread's columns [32c, 32c + 32) of the pass
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 o;
            __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
            for (int j = 0; j < 4; ++j) o2[j] = __floats2bfloat162_rn(v[q * 8 + 2 * j], v[q * 8 + 2 * j + 1]);
            *reinterpret_cast<uint4*>(stage_row + (((c * 4 + q) ^ (lane & 7)) << 4)) = o;
          }
        };
#pragma unroll 1
        for (int pass = 0; pass < 2; ++pass) {
          const int coff = part * 128 + pass * 64;              // column offset inside the tile
          const int colbase = n0 + coff;
          if (ep.pre != nullptr && (ep.act == 1 || ep.gate != nullptr)) {
            // second output first (TMEM is read again below): the pre-activation of a GELU, or the plain product of a
            // gated-residual GEMM (training keeps it for the gate gradient)
#pragma unroll 1
            for (int c = 0; c < 2; ++c) {
              uint32_t r[32];
              tmem_ld32(t_row + coff + c * 32, r);
              tmem_ld_wait();
              float v[32];
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
              if (ep.bias != nullptr) {
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] += __bfloat162float(ep.bias[colbase + c * 32 + j]);
              }
              stage_chunk(c, v);
            }
            write_out(ep.pre, colbase);
          }
          if (ep.gate != nullptr) {                             // residual rows in, coalesced
#pragma unroll 4
            for (int it = 0; it < 8; ++it) {
              const int r_src = it * 4 + (lane >> 3), chunk = lane & 7;
              uint4 v4 = make_uint4(0, 0, 0, 0);
              if (row0 + r_src < M) v4 = *reinterpret_cast<const uint4*>(ep.resid + (size_t)(row0 + r_src) * N + colbase + chunk * 8);
              *reinterpret_cast<uint4*>(stage_warp + r_src * 128 + ((chunk ^ (r_src & 7)) << 4)) = v4;
            }
            __syncwarp();
          }
#pragma unroll 1
          for (int c = 0; c < 2; ++c) {
            uint32_t r[32];
            tmem_ld32(t_row + coff + c * 32, r);
            tmem_ld_wait();
            float v[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
            const int col0 = colbase + c * 32;
            if (ep.bias != nullptr) {
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] += __bfloat162float(ep.bias[col0 + j]);
            }
            if (ep.act == 1) {
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] = gelu_erf(v[j]);
            }
            if (ep.gate != nullptr) {
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const uint4 rr = *reinterpret_cast<const uint4*>(stage_row + (((c * 4 + q) ^ (lane & 7)) << 4));
                const __nv_bfloat162* r2 = reinterpret_cast<const __nv_bfloat162*>(&rr);
                float g[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                if (gate_row != nullptr) {
                  const float4 g0 = *reinterpret_cast<const float4*>(gate_row + col0 + q * 8);
                  const float4 g1 = *reinterpret_cast<const float4*>(gate_row + col0 + q * 8 + 4);
                  g[0] = g0.x; g[1] = g0.y; g[2] = g0.z; g[3] = g0.w; g[4] = g1.x; g[5] = g1.y; g[6] = g1.z; g[7] = g1.w;
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const float2 rf = __bfloat1622float2(r2[j]);
                  v[q * 8 + 2 * j] = rf.x + g[2 * j] * v[q * 8 + 2 * j];
                  v[q * 8 + 2 * j + 1] = rf.y + g[2 * j + 1] * v[q * 8 + 2 * j + 1];
                }
              }
            }
            stage_chunk(c, v);                                  // in place: a thread only ever touches its own row here
          }
          write_out(ep.C, colbase);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          if (CTA2) mbar_arrive_cluster(acc_empty_leader[acc]);
          else mbar_arrive(&acc_empty[acc]);
        }
        if (++acc == 2) { acc = 0; acc_ph ^= 1; }
        continue;
      }
#pragma unroll 1
      for (int c = part * 4; c < part * 4 + 4; ++c) {
        uint32_t r[32];
        tmem_ld32(t_row + c * 32, r);
        tmem_ld_wait();
        const int col0 = n0 + c * 32;
        if (row < M && col0 < N) {
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
          const bool full_chunk = vec_ok && (col0 + 32 <= N);
          const size_t off = (size_t)row * N + col0;
          if (ep.bias != nullptr) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (full_chunk || col0 + j < N) v[j] += __bfloat162float(ep.bias[col0 + j]);
          }
          if (ep.act == 1) {
            if (ep.pre != nullptr) {
              if (full_chunk) {
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                  uint4 o;
                  __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
                  for (int j = 0; j < 4; ++j) o2[j] = __floats2bfloat162_rn(v[q * 8 + 2 * j], v[q * 8 + 2 * j + 1]);
                  *reinterpret_cast<uint4*>(ep.pre + off + q * 8) = o;
                }
              } else {
                for (int j = 0; j < 32 && col0 + j < N; ++j) ep.pre[off + j] = __float2bfloat16(v[j]);
              }
            }
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = gelu_erf(v[j]);
          }
          if (gate_row != nullptr) {
            if (full_chunk) {
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const uint4 rr = *reinterpret_cast<const uint4*>(ep.resid + off + q * 8);
                const __nv_bfloat162* r2 = reinterpret_cast<const __nv_bfloat162*>(&rr);
                const float4 g0 = *reinterpret_cast<const float4*>(gate_row + col0 + q * 8);
                const float4 g1 = *reinterpret_cast<const float4*>(gate_row + col0 + q * 8 + 4);
                const float g[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const float2 rf = __bfloat1622float2(r2[j]);
                  v[q * 8 + 2 * j] = rf.x + g[2 * j] * v[q * 8 + 2 * j];
                  v[q * 8 + 2 * j + 1] = rf.y + g[2 * j + 1] * v[q * 8 + 2 * j + 1];
                }
              }
            } else {
              for (int j = 0; j < 32 && col0 + j < N; ++j)
                v[j] = __bfloat162float(ep.resid[off + j]) + gate_row[col0 + j] * v[j];
            }
          }
          if (full_chunk) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              uint4 o;
              __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
              for (int j = 0; j < 4; ++j) o2[j] = __floats2bfloat162_rn(v[q * 8 + 2 * j], v[q * 8 + 2 * j + 1]);
              *reinterpret_cast<uint4*>(ep.C + off + q * 8) = o;
            }
          } else {
            for (int j = 0; j < 32 && col0 + j < N; ++j) ep.C[off + j] = __float2bfloat16(v[j]);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
          if (CTA2) mbar_arrive_cluster(acc_empty_leader[acc]);
          else mbar_arrive(&acc_empty[acc]);
        }
      if (++acc == 2) { acc = 0; acc_ph ^= 1; }
    }
    if (!ok && lane == 0) { atomicCAS(err, 0, 3); *abort_flag = 1; }
  }

  // ---------------------------------------------------------------------- teardown
  __syncwarp();
  if (*abort_flag) {
    // let outstanding bulk copies / MMAs drain before shared memory and TMEM go away
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (CTA2) cluster_sync_all();      // neither CTA leaves (or frees TMEM) while the other may still signal it or read its tiles
  if (warp == 1) {
    tc_fence_after();
    if (CTA2) tmem_dealloc_pair(tmem_base, 512);
    else tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace cb200

using namespace cb200;

template <int A_MN, int B_MN, bool GATHER = false>
static int launch_gemm(const void* A, const void* B, int M, int N, int K, const GemmEpilogue& ep, int* err, int sms,
                       cudaStream_t st, const GatherB& gb = GatherB{}) {
  CUtensorMap ta, tb;
  int rc;
  // A: K-major [M,K] -> dims {K, M}, box {64, 128};  MN-major stored [K,M] -> dims {M, K}, box {64, 64}
  if (A_MN == 0) rc = make_tmap_2d_bf16(&ta, A, (uint64_t)K, (uint64_t)M, (uint64_t)K * 2, BK, BM);
  else rc = make_tmap_2d_bf16(&ta, A, (uint64_t)M, (uint64_t)K, (uint64_t)M * 2, 64, BK);
  if (rc) return rc;
  if (B_MN == 0) rc = make_tmap_2d_bf16(&tb, B, (uint64_t)K, (uint64_t)N, (uint64_t)K * 2, BK, BN);
  else rc = make_tmap_2d_bf16(&tb, B, (uint64_t)N, (uint64_t)K, (uint64_t)N * 2, 64, BK);
  if (rc) return rc;
  static bool attr_set = false;      // one flag per template instantiation
  auto kern = gemm_bf16_kernel<A_MN, B_MN, GATHER>;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
    if (e != cudaSuccess) return 100 + (int)e;
    attr_set = true;
  }
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  // with a gather every SM takes part (its gather warps work even when it has no tile): the grid is the whole machine
  const int grid = GATHER ? sms : (tiles < sms ? tiles : sms);
  kern<<<grid, kGemmThreads + (GATHER ? kGatherWarps * 32 : 0), kSmemBytes, st>>>(ta, tb, M, N, K, ep, gb, err);
  return (int)cudaGetLastError();
}

// Same contraction on CTA pairs (template flag CTA2): clusters of two CTAs, one 256 x 256 tile per pair.
template <int A_MN, int B_MN>
static int launch_gemm_pair(const void* A, const void* B, int M, int N, int K, const GemmEpilogue& ep, int* err, int sms,
                            cudaStream_t st) {
  CUtensorMap ta, tb;
  int rc;
  if (A_MN == 0) rc = make_tmap_2d_bf16(&ta, A, (uint64_t)K, (uint64_t)M, (uint64_t)K * 2, BK, BM);
  else rc = make_tmap_2d_bf16(&ta, A, (uint64_t)M, (uint64_t)K, (uint64_t)M * 2, 64, BK);
  if (rc) return rc;
  if (B_MN == 0) rc = make_tmap_2d_bf16(&tb, B, (uint64_t)K, (uint64_t)N, (uint64_t)K * 2, BK, BN / 2);   // each CTA loads half the columns
  else rc = make_tmap_2d_bf16(&tb, B, (uint64_t)N, (uint64_t)K, (uint64_t)N * 2, 64, BK);
  if (rc) return rc;
  static bool attr_set = false;
  auto kern = gemm_bf16_kernel<A_MN, B_MN, false, true>;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
    if (e != cudaSuccess) return 100 + (int)e;
    attr_set = true;
  }
  const int tiles = ((M + 2 * BM - 1) / (2 * BM)) * ((N + BN - 1) / BN);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * (sms / 2));
  cfg.blockDim = dim3(kGemmThreads);
  cfg.dynamicSmemBytes = kSmemBytes;
  cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = 2;
  at[0].val.clusterDim.y = 1;
  at[0].val.clusterDim.z = 1;
  cfg.attrs = at;
  cfg.numAttrs = 1;
  // A persistent grid must be resident as a whole: the pairs that the GPU can hold at once (a pair lives inside one GPC, so a
  // GPC with an odd number of free SMs leaves one out) bound the grid, otherwise late pairs would run after the others.
  static int max_pairs = 0;
  if (max_pairs == 0) {
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n < 1) return 600;
    max_pairs = n;
  }
  const int pairs = std::min(tiles, std::min(max_pairs, sms / 2));
  cfg.gridDim = dim3(2 * pairs);
  const cudaError_t e = cudaLaunchKernelEx(&cfg, kern, ta, tb, M, N, K, ep, GatherB{}, err);
  return e == cudaSuccess ? 0 : 500 + (int)e;
}

// 0: single-CTA tiles; 1 (default): CTA pairs where the shape allows (measured 8-45 % faster on the 2B shapes: half the B-operand
// bytes per CTA). COSMOS_B200_GEMM_PAIR=0 selects single-CTA tiles; cb200_gemm_pair_mode switches at run time (the kernel
// benchmark compares the two).
static int g_pair_mode = -1;
extern "C" int cb200_gemm_pair_mode(int mode) {
  if (g_pair_mode < 0) {
    const char* e = getenv("COSMOS_B200_GEMM_PAIR");
    g_pair_mode = (e != nullptr && e[0] == '0') ? 0 : 1;
  }
  const int prev = g_pair_mode;
  if (mode >= 0) g_pair_mode = mode;
  return prev;
}

extern "C" int cb200_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, int a_mn, int b_mn,
                               const void* bias, int act, void* pre, const void* resid, const float* gate, int L, int* err,
                               int sms, cudaStream_t st) {
  GemmEpilogue ep{};
  ep.C = (bf16*)C;
  ep.pre = (bf16*)pre;
  ep.bias = (const bf16*)bias;
  ep.resid = (const bf16*)resid;
  ep.gate = gate;
  ep.act = act;
  ep.L = L > 0 ? L : 1;
  if (cb200_gemm_pair_mode(-1) == 1 && M >= 2 * BM && N % 8 == 0) {
    if (a_mn == 0 && b_mn == 0) return launch_gemm_pair<0, 0>(A, B, M, N, K, ep, err, sms, st);
    if (a_mn == 0 && b_mn == 1) return launch_gemm_pair<0, 1>(A, B, M, N, K, ep, err, sms, st);
    if (a_mn == 1 && b_mn == 0) return launch_gemm_pair<1, 0>(A, B, M, N, K, ep, err, sms, st);
    return launch_gemm_pair<1, 1>(A, B, M, N, K, ep, err, sms, st);
  }
  if (a_mn == 0 && b_mn == 0) return launch_gemm<0, 0>(A, B, M, N, K, ep, err, sms, st);
  if (a_mn == 0 && b_mn == 1) return launch_gemm<0, 1>(A, B, M, N, K, ep, err, sms, st);
  if (a_mn == 1 && b_mn == 0) return launch_gemm<1, 0>(A, B, M, N, K, ep, err, sms, st);
  return launch_gemm<1, 1>(A, B, M, N, K, ep, err, sms, st);
}

// C is not written: row (b, s) of A[M = B*S, K] @ W[N = H*128, K]^T is split into heads, each head is RMS-normalised with
// `norm_w` (optional), rotated by cos/sin [S, 64] (optional, needs norm_w) and stored into staging buffer ptrs[head / Hl] at
// [b, rank * S + s, head % Hl, :].  The buffers may live on peer GPUs (plain stores over NVLink).
extern "C" int cb200_gemm_bf16_scatter_heads(const void* A, const void* W, int M, int N, int K, const int64_t* ptrs, int P,
                                             int rank, int S, const float* norm_w, const float* cosv, const float* sinv,
                                             float eps, void* raw, float* rstd_out, int* err, int sms, cudaStream_t st) {
  if (P < 1 || P > 8 || N % 128 != 0 || (N / 128) % P != 0 || S <= 0 || M % S != 0) return -21;
  if (cosv != nullptr && norm_w == nullptr) return -22;
  if ((raw != nullptr) != (rstd_out != nullptr) || (raw != nullptr && norm_w == nullptr)) return -23;
  GemmEpilogue ep{};
  for (int i = 0; i < P; ++i) ep.hs.ptrs[i] = ptrs[i];
  ep.hs.w = norm_w;
  ep.hs.cosv = cosv;
  ep.hs.sinv = sinv;
  ep.hs.S = S;
  ep.hs.Hl = (N / 128) / P;
  ep.hs.P = P;
  ep.hs.rank = rank;
  ep.hs.eps = eps;
  ep.hs.raw = (bf16*)raw;
  ep.hs.rstd_out = rstd_out;
  ep.L = 1;
  if (cb200_gemm_pair_mode(-1) == 1 && M >= 2 * BM) return launch_gemm_pair<0, 0>(A, W, M, N, K, ep, err, sms, st);
  return launch_gemm<0, 0>(A, W, M, N, K, ep, err, sms, st);
}

// C = epilogue(A @ op(W)) where W [rows, ld] is sharded by rows over P ranks (rank r: shard_ptrs[r] holds rows [r * chunk_rows, ...)).
// b_mn = 0: forward, C[M, rows] = A[M, ld] @ W^T; b_mn = 1: dgrad, C[M, ld] = A[M, rows] @ W. `ws` [rows, ld] receives the gathered
// weight (and stays valid after the call); `counters`: ceil(rows / 256) ints of scratch.
extern "C" int cb200_gemm_bf16_gather(const void* A, void* ws, void* C, int M, int rows, int ld, int b_mn, const int64_t* shard_ptrs,
                                      int P, int chunk_rows, int* counters, const void* bias, int act, void* pre, int* err, int sms,
                                      cudaStream_t st) {
  if (P < 1 || P > 8 || chunk_rows < 1 || (long)chunk_rows * P < rows || ld % 8 != 0) return -31;
  GemmEpilogue ep{};
  ep.C = (bf16*)C;
  ep.pre = (bf16*)pre;
  ep.bias = (const bf16*)bias;
  ep.act = act;
  ep.L = 1;
  GatherB gb{};
  for (int i = 0; i < P; ++i) gb.ptrs[i] = shard_ptrs[i];
  gb.ws = (bf16*)ws;
  gb.counters = counters;
  gb.P = P;
  gb.chunk_rows = chunk_rows;
  gb.rows = rows;
  gb.ld = ld;
  const int n_groups = (rows + kGatherGroupRows - 1) / kGatherGroupRows;
  gb.slices = sms / n_groups < 1 ? 1 : (sms / n_groups > 16 ? 16 : sms / n_groups);
  cudaError_t e = cudaMemsetAsync(counters, 0, (size_t)n_groups * sizeof(int), st);
  if (e != cudaSuccess) return 400 + (int)e;
  if (b_mn == 0) return launch_gemm<0, 0, true>(A, ws, M, rows, ld, ep, err, sms, st, gb);
  return launch_gemm<0, 1, true>(A, ws, M, ld, rows, ep, err, sms, st, gb);
}
