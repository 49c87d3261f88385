// Flash attention forward on tcgen05 / TMEM (sm_100a), head_dim 128, bf16, non-causal.
//
// One CTA owns two 128-row query tiles of one (batch, head) and walks over the keys in tiles of 128:
//
//   warps 0-3   softmax of query tile 0   (thread i <-> query row i <-> TMEM lane i)
//   warps 4-7   softmax of query tile 1
//   warp  8     TMA producer: Q once, then K_0 V_0 K_1 V_1 ... through one 5-slot ring (128-byte swizzle)
//   warp  9     MMA issuer (one thread): S_t = Q_t K_j^T  (SS form, both operands K-major in smem)
//                                        O_t += P_t V_j   (TS form: P read from TMEM, V N-major in smem)
//
// TMEM (512 columns): S_0 [0,128) S_1 [128,256) fp32 scores, O_0 [256,384) O_1 [384,512) fp32 outputs.
// The softmax thread pulls its whole score row into registers with four tcgen05.ld, and writes the bf16
// probabilities back over the first 64 columns of the same S buffer with tcgen05.st; the P.V MMA takes
// them from there, so probabilities never visit shared memory. While one tile is in softmax the tensor
// core runs the other tile's P.V and next Q.K^T (ping-pong).
//
// Register budget decides the shape of this kernel: one thread per query row holds the whole 128-column score row.
//
// Three pipes are needed for exactly the same time per 128 x 128 tile at full rate - the tensor pipe (2 x 512 clocks), the
// exponential unit (16,384 ex2 at 16 per clock) and, for the Q.K^T half, shared-memory operand bandwidth - so the kernel is
// tuned by taking work off the exponential unit and by shortening the softmax -> MMA hand-off:
//   * EXPM of every 4 element pairs compute 2^x on the FMA pipe instead (round-to-nearest split, degree-3 polynomial in
//     packed fp32x2 arithmetic, exponent add; relative error 1e-4, a twentieth of a bf16 half-ulp);
//   * the row maximum uses the three-input max;
//   * SPLITP = 2 or 4: the probabilities are published in halves / quarters of the key tile on their own barriers, so P.V of
//     the first keys runs while the rest of the row is still being exponentiated.
// QT = 1 is the shape for short key sequences (cross-attention, 512 keys): one query tile, 192 threads, 97 KB of shared memory and 256
// TMEM columns per CTA, so that two CTAs share an SM and fill each other's prologue / epilogue gaps.
//
// Online softmax keeps a reference maximum per row that is only moved when the running maximum grows
// by more than 2^8; the output accumulator is rescaled in TMEM only then (rare after the first tiles).
// All waits are bounded and report through `err`.

#include <math.h>

#include "common.cuh"
#include "launchers.h"
#include "sm100.cuh"
#include "tmap.h"

namespace cb200 {
using namespace sm100;

namespace fa {
constexpr int HD = 128;          // head dim
constexpr int BQ = 128;          // query rows per tile (two tiles per CTA)
constexpr int BKV = 128;         // keys per tile
constexpr int kTileBytes = 128 * HD * 2;  // 32 KB
constexpr int kHalfBytes = kTileBytes / 2;
constexpr float kRescaleThreshold = 8.0f;  // log2 units
// shape of a CTA with QT query tiles: 4 softmax warps per tile, then the TMA warp and the MMA warp
// REGS: the CTA is padded to whole warpgroups (12 warps) and re-divides its registers at start: the warpgroup of the TMA / MMA warps
// gives registers back (setmaxnreg.dec) and the softmax warpgroups take them (setmaxnreg.inc), which removes the spills of the
// 128-value score row. The padding also pays for a second MMA issuer: each query tile gets its own issuing warp, so a wait
// on one tile's probabilities never delays the other tile's MMAs.
template <int QT, bool REGS = false>
struct Shape {
  static constexpr int kRing = QT == 2 ? 5 : 2;           // K/V ring slots
  static constexpr int kTmaWarp = 4 * QT, kMmaWarp = 4 * QT + 1;
  static constexpr int kIssuers = REGS ? QT : 1;          // MMA issuer warps kMmaWarp .. kMmaWarp + kIssuers - 1
  static constexpr int kThreads = REGS ? (4 * QT + 4) * 32 : (4 * QT + 2) * 32;
  // register re-division: launched with kRegsLaunch per thread (12 warps); the CTA can only re-divide that allocation
  static constexpr int kRegsLaunch = 168, kRegsSoftmax = 224, kRegsOther = 56;
  static_assert(!REGS || (8 * kRegsSoftmax + 4 * kRegsOther <= 12 * kRegsLaunch), "setmaxnreg budget: increases must be covered by decreases");
  static constexpr int kMinCtas = QT == 2 ? 1 : 2;
  static constexpr uint32_t kTmemCols = 256 * QT;
  static constexpr size_t kSmem = (QT + kRing) * (size_t)kTileBytes + 1024 + 256;
};
}  // namespace fa

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// 2^x for a pair of values, x <= ~100, on the FMA / ALU pipes: t = x + 1.5 * 2^23 rounds x to the nearest integer n (kept in
// the low mantissa bits of t), f = x - n lies in [-0.5, 0.5], 2^f comes from a degree-3 polynomial fitted for a relative
// error of 1.0e-4, and n is added to the exponent field (t << 23 drops everything but n; x is clamped at -126 so that the
// result stays a normal number). Packed fp32x2 instructions halve the issue slots of the six additions / multiply-adds.
__device__ __forceinline__ float2 exp2_poly2(float2 x) {
  x.x = fmaxf(x.x, -126.f);
  x.y = fmaxf(x.y, -126.f);
  const float2 magic = make_float2(12582912.f, 12582912.f);
  const float2 t = add2(x, magic);
  const float2 n = add2(t, make_float2(-12582912.f, -12582912.f));
  const float2 f = fma2(n, make_float2(-1.f, -1.f), x);
  float2 p = fma2(f, make_float2(0.05500893f, 0.05500893f), make_float2(0.24221095f, 0.24221095f));
  p = fma2(p, f, make_float2(0.6932829f, 0.6932829f));
  p = fma2(p, f, make_float2(1.f, 1.f));
  float2 r;
  r.x = __int_as_float(__float_as_int(p.x) + (__float_as_int(t.x) << 23));
  r.y = __int_as_float(__float_as_int(p.y) + (__float_as_int(t.y) << 23));
  return r;
}

__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

// Ulysses head->sequence exchange fused into the output store: this rank holds heads [rank*H, rank*H + H) of the whole
// sequence (Sq = P * S_loc rows); row s of the output belongs to rank s / S_loc and is stored straight into that rank's buffer
// [B, S_loc, P*H, 128] (plain 16-byte stores, local or over NVLink).  P == 0: the output goes to O as usual.
struct SeqScatter {
  int64_t ptrs[8];
  int P, rank, S_loc;
};

// Neighbourhood (tile-sparse) attention.  The sequence is a T x H x W token grid in its natural (t, h, w) order; the kernel
// works on 4 x 4 x 8 (t, h, w) tiles of it, which TMA fetches as 5-D boxes {64 channels, 1 head, 8 w, 4 h, 4 t} straight from
// that layout (the 128 rows land in shared memory in (t, h, w) order of the tile, the same layout a [128, 64] box has), so no
// re-ordering pass is needed; "row" below means the position in tile order: tile index * 128 + position in the tile, tiles
// in (tile_t, tile_h, tile_w) row-major order.  A CTA (two query tiles) visits only
// the key tiles of its list; inside a visited tile a key is visible to a query iff it is visible along each axis, which
// three byte tables give: bit i of bt[t_query * nT + tile_t_key] says whether key plane i of that tile is visible, etc.
struct NaParams {
  const int* kv_idx;        // [n_blocks, max_n] key-tile indices per query block (ascending), nullptr: dense attention
  const int* kv_cnt;        // [n_blocks] >= 1
  const uint8_t* bt;        // [T, nT]
  const uint8_t* bh;        // [H, nH]
  const uint8_t* bw;        // [W, nW]
  int max_n, nT, nH, nW;
};

template <int QT, int EXPM, int SPLITP, bool NA, bool REGS>
__global__ void __launch_bounds__(fa::Shape<QT, REGS>::kThreads, fa::Shape<QT, REGS>::kMinCtas)
fa_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
              const __grid_constant__ CUtensorMap tm_v, bf16* __restrict__ O, float* __restrict__ LSE, int Sq, int Skv, int H,
              float scale_log2, SeqScatter sc, NaParams na, int* __restrict__ err) {
  using namespace fa;
  using Sh = Shape<QT, REGS>;
  constexpr int kRing = Sh::kRing, kMmaWarp = Sh::kMmaWarp, kTmaWarp = Sh::kTmaWarp;
  static_assert(!REGS || QT == 2, "register re-division needs whole warpgroups per role");
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = smem;                      // QT tiles
  uint8_t* sR = smem + QT * kTileBytes;    // ring of kRing tiles: K_0 V_0 K_1 V_1 ...
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (QT + kRing) * kTileBytes);
  uint64_t* q_full = bars;                 // [1]
  uint64_t* r_full = bars + 1;             // [kRing]
  uint64_t* r_empty = bars + 1 + kRing;    // [kRing]
  uint64_t* s_full = bars + 1 + 2 * kRing; // [QT]  scores of tile t ready (also: all earlier MMAs complete)
  uint64_t* p_ready = s_full + QT;         // [QT]  probabilities of tile t written to TMEM
  uint64_t* p_part = p_ready + QT;         // [QT][3] probabilities of the first 1, 2, 3 key quarters of tile t written (SPLITP > 1)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(p_part + 3 * QT);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  // the shuffle makes the warp index (and every role branch below) provably warp-uniform for the compiler
  const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;
  const int h = blockIdx.y, b = blockIdx.z;
  const int q_base = blockIdx.x * QT * BQ;
  const int n_kv = NA ? na.kv_cnt[blockIdx.x] : (Skv + BKV - 1) / BKV;
  const int* kv_list = NA ? na.kv_idx + (size_t)blockIdx.x * na.max_n : nullptr;
  constexpr uint32_t kOBase = QT * 128;    // TMEM: S_t at t * 128, O_t at kOBase + t * 128

  // A CTA that starts after another one has reported an error leaves at once (the whole grid then drains in microseconds
  // instead of running every CTA into its own wait limit). One thread reads the word so that the decision is CTA-uniform.
  if (threadIdx.x == 0) *abort_flag = *reinterpret_cast<volatile int*>(err);
  __syncthreads();
  if (*abort_flag != 0) return;
  __syncthreads();
  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < kRing; ++i) {
      mbar_init(&r_full[i], 1);
      mbar_init(&r_empty[i], Sh::kIssuers);   // every issuer has finished reading the slot
    }
    for (int i = 0; i < QT; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&p_ready[i], 4);
      for (int k = 0; k < 3; ++k) mbar_init(&p_part[i * 3 + k], 4);
    }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == kMmaWarp) {
    tmem_alloc(tmem_slot, Sh::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // With REGS every role branch starts by re-dividing the registers of its warpgroup (the instruction has to sit inside the
  // branch: the compiler takes the smallest limit that reaches a join point as the limit of everything after it).
  if (warp == kTmaWarp) {
    // -------------------------------------------------------------------- TMA producer
    if (REGS) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(Sh::kRegsOther));
    if (lane == 0) {
      prefetch_tmap(&tm_q);
      prefetch_tmap(&tm_k);
      prefetch_tmap(&tm_v);
      mbar_arrive_expect_tx(q_full, QT * kTileBytes);
      // neighbourhood mode: tile index -> coordinates of its 5-D box (w0, h0, b * T + t0)
      auto load_tile = [&](uint8_t* dst, const CUtensorMap* tm, uint64_t* bar, int tile) {
        if (NA) {
          const int iT = tile / (na.nH * na.nW), iH = (tile / na.nW) % na.nH, iW = tile % na.nW;
          for (int c = 0; c < 2; ++c) tma_load_5d(dst + c * kHalfBytes, tm, bar, c * 64, h, iW * 8, iH * 4, b * (na.nT * 4) + iT * 4);
        } else {
          for (int c = 0; c < 2; ++c) tma_load_4d(dst + c * kHalfBytes, tm, bar, c * 64, h, tile * BKV, b);
        }
      };
      for (int t = 0; t < QT; ++t) load_tile(sQ + t * kTileBytes, &tm_q, q_full, blockIdx.x * QT + t);
      bool ok = true;
      int slot = 0;
      uint32_t ph = 0;
      for (int n = 0; n < 2 * n_kv; ++n) {  // even n: K_{n/2}, odd n: V_{n/2}
        if (!mbar_wait(&r_empty[slot], ph ^ 1, abort_flag)) { ok = false; break; }
        mbar_arrive_expect_tx(&r_full[slot], kTileBytes);
        const CUtensorMap* tm = (n & 1) ? &tm_v : &tm_k;
        load_tile(sR + slot * kTileBytes, tm, &r_full[slot], NA ? kv_list[n >> 1] : (n >> 1));
        if (++slot == kRing) { slot = 0; ph ^= 1; }
      }
      if (!ok) { atomicCAS(err, 0, 11); *abort_flag = 1; }
    }
  } else if (warp >= kMmaWarp && warp < kMmaWarp + Sh::kIssuers) {
    // -------------------------------------------------------------------- MMA issuer(s): tiles [t_lo, t_hi) of this warp
    if (REGS) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(Sh::kRegsOther));
    const int t_lo = Sh::kIssuers == 1 ? 0 : warp - kMmaWarp, t_hi = Sh::kIssuers == 1 ? QT : t_lo + 1;
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
      // O_t += P_t[:, 16 kk0 .. 16 kk1) V[16 kk0 .. 16 kk1, :]
      auto issue_pv = [&](int t, int slot, bool accumulate, int kk0, int kk1) {
        const uint64_t bv = dR_mn + (uint64_t)(slot * (kTileBytes >> 4));
#pragma unroll
        for (int kk = kk0; kk < kk1; ++kk) {
          umma_ts_w(tmem_base + kOBase + t * 128, tmem_base + t * 128 + kk * 8, bv + (uint32_t)(kk * (2048 >> 4)), idesc_pv,
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
        for (int t = t_lo; t < t_hi; ++t) {
          issue_qk(t, slot);
          umma_commit_w(&s_full[t], leader);
        }
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
        for (int t = t_lo; t < t_hi; ++t) {
          if (SPLITP > 1) {
            // the softmax publishes its row in SPLITP parts; P.V follows part by part
            constexpr int kPer = 8 / SPLITP;
#pragma unroll
            for (int part = 0; part < SPLITP; ++part) {
              uint64_t* bar = part == SPLITP - 1 ? &p_ready[t] : &p_part[t * 3 + (part + 1) * (4 / SPLITP) - 1];
              if (!wait_all(bar, j & 1)) { ok = false; break; }
              tc_fence_after();
              issue_pv(t, v_slot, j > 0 || part > 0, part * kPer, (part + 1) * kPer);
            }
            if (!ok) break;
          } else {
            if (!wait_all(&p_ready[t], j & 1)) { ok = false; break; }
            tc_fence_after();
            issue_pv(t, v_slot, j > 0, 0, 8);
          }
          if (t == t_hi - 1) umma_commit_w(&r_empty[v_slot], leader);
          if (has_next) issue_qk(t, k_slot);
          if (t == t_hi - 1 && has_next) umma_commit_w(&r_empty[k_slot], leader);
          umma_commit_w(&s_full[t], leader);
        }
      }
      if (!ok && lane == 0) { atomicCAS(err, 0, 12); *abort_flag = 1; }
    }
  } else if (warp < 4 * QT) {
    // -------------------------------------------------------------------- softmax warpgroups
    if (REGS) asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(Sh::kRegsSoftmax));
    const int t = warp >> 2;       // query tile
    const int quarter = warp & 3;  // TMEM lane quarter
    const int q_row = q_base + t * BQ + quarter * 32 + lane;
    const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
    const uint32_t tS = tmem_base + t * 128 + lane_off;
    const uint32_t tO = tmem_base + kOBase + t * 128 + lane_off;
    float m_ref = -INFINITY;  // reference maximum used in the exponent (log2 domain)
    float l = 0.f;
    bool ok = true;
    // neighbourhood mode: rows of the byte tables that belong to this query (clamped for rows past the sequence end)
    const uint8_t *row_bt = nullptr, *row_bh = nullptr, *row_bw = nullptr;
    if (NA) {
      const int qr = q_row < Sq ? q_row : Sq - 1;
      const int qt = qr >> 7, loc = qr & 127;
      const int qT = qt / (na.nH * na.nW), qH = (qt / na.nW) % na.nH, qW = qt % na.nW;
      row_bt = na.bt + (size_t)(qT * 4 + (loc >> 5)) * na.nT;
      row_bh = na.bh + (size_t)(qH * 4 + ((loc >> 3) & 3)) * na.nH;
      row_bw = na.bw + (size_t)(qW * 8 + (loc & 7)) * na.nW;
    }
    for (int j = 0; j < n_kv; ++j) {
      uint32_t vis[4] = {0xffffffffu, 0xffffffffu, 0xffffffffu, 0xffffffffu};  // visibility of the 128 keys of this tile
      if (NA) {
        const int kt = kv_list[j];
        const uint32_t mt = row_bt[kt / (na.nH * na.nW)], mh = row_bh[(kt / na.nW) % na.nH], mw = row_bw[kt % na.nW];
        uint32_t plane = 0;                       // 32 keys of one t-plane: bit (lh * 8 + lw)
#pragma unroll
        for (int lh = 0; lh < 4; ++lh) plane |= ((mh >> lh) & 1u) ? (mw << (8 * lh)) : 0u;
#pragma unroll
        for (int c = 0; c < 4; ++c) vis[c] = ((mt >> c) & 1u) ? plane : 0u;
      }
      if (!mbar_wait(&s_full[t], j & 1, abort_flag)) { ok = false; break; }
      tc_fence_after();
      uint32_t r[4][32];
      tmem_ld32(tS, r[0]);
      tmem_ld32(tS + 32, r[1]);
      tmem_ld32(tS + 64, r[2]);
      tmem_ld32(tS + 96, r[3]);
      tmem_ld_wait();
      const int n_valid = NA ? BKV : Skv - j * BKV;   // neighbourhood mode works on whole tiles
      if (n_valid < BKV) {
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (c * 32 + i >= n_valid) r[c][i] = 0xff800000u;  // -inf
      }
      if (NA && __any_sync(0xffffffffu, (vis[0] & vis[1] & vis[2] & vis[3]) != 0xffffffffu)) {
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (!((vis[c] >> i) & 1u)) r[c][i] = 0xff800000u;
      }
      // row maximum: four independent chains of three-input max instructions
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int i = 0; i < 32; i += 2) mx4[(i >> 1) & 3] = max3(mx4[(i >> 1) & 3], __uint_as_float(r[c][i]), __uint_as_float(r[c][i + 1]));
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * scale_log2;
      const bool need = mx > m_ref + kRescaleThreshold;
      float alpha = 1.f;
      if (need) {
        alpha = (m_ref == -INFINITY) ? 0.f : ex2(m_ref - mx);
        m_ref = mx;
        l *= alpha;
      }
      if (j > 0 && __any_sync(0xffffffffu, need)) {
        // rescale the output accumulator of this warp's 32 rows in TMEM
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t o[32];
          tmem_ld32(tO + c * 32, o);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tmem_st32(tO + c * 32, o);
        }
        tmem_st_wait();
      }
      // probabilities -> bf16 pairs over the first 64 columns of the score buffer
      // a row that has seen no visible key yet keeps m_ref = -inf: use 0 so that its masked scores give exp2(-inf) = 0
      const float neg_m = (NA && m_ref == -INFINITY) ? 0.f : -m_ref;
      const float2 sc2 = make_float2(scale_log2, scale_log2), nm2 = make_float2(neg_m, neg_m);
      float2 lsum2 = make_float2(0.f, 0.f);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float2 x = fma2(make_float2(__uint_as_float(r[c][2 * i]), __uint_as_float(r[c][2 * i + 1])), sc2, nm2);
          float2 p;
          if ((i & 3) < EXPM) {
            p = exp2_poly2(x);
          } else {
            p.x = ex2(x.x);
            p.y = ex2(x.y);
          }
          lsum2 = add2(lsum2, p);
          __nv_bfloat162 pb = __floats2bfloat162_rn(p.x, p.y);
          pk[i] = *reinterpret_cast<uint32_t*>(&pb);
        }
        tmem_st16(tS + c * 16, pk);
        if (SPLITP > 1 && c < 3 && ((c + 1) % (4 / SPLITP)) == 0) {
          tmem_st_wait();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&p_part[t * 3 + c]);
        }
      }
      l += lsum2.x + lsum2.y;
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_ready[t]);
    }
    if (ok) ok = mbar_wait(&s_full[t], n_kv & 1, abort_flag);
    if (ok) {
      tc_fence_after();
      const float inv_l = 1.f / l;
      int out_row = q_row;   // position of this query in the output sequence
      if (NA && q_row < Sq) {
        const int qt = q_row >> 7, loc = q_row & 127;
        const int tq = (qt / (na.nH * na.nW)) * 4 + (loc >> 5), hq = ((qt / na.nW) % na.nH) * 4 + ((loc >> 3) & 3), wq = (qt % na.nW) * 8 + (loc & 7);
        out_row = (tq * (na.nH * 4) + hq) * (na.nW * 8) + wq;
      }
      bf16* orow = O + (((size_t)b * Sq + out_row) * H + h) * HD;
      if (sc.P > 0 && q_row < Sq) {
        const int dst = q_row / sc.S_loc, s_loc = q_row - dst * sc.S_loc;
        orow = reinterpret_cast<bf16*>(sc.ptrs[dst]) + (((size_t)b * sc.S_loc + s_loc) * (sc.P * H) + sc.rank * H + h) * HD;
      }
      // The finished rows go through shared memory (this tile's Q buffer is free: its last Q.K^T has completed) so that the
      // global stores are coalesced: 16 lanes cover one 256-byte row, a warp store is two contiguous 256-byte segments.
      // That matters most when the destination is a peer's memory: NVLink moves 256-byte writes far better than 16-byte ones.
      uint8_t* stage_warp = sQ + t * kTileBytes + quarter * (32 * 256);
      uint8_t* stage_row = stage_warp + lane * 256;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t o[32];
        tmem_ld32(tO + c * 32, o);
        tmem_ld_wait();
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          uint4 ov;
          __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
          for (int i = 0; i < 4; ++i)
            o2[i] = __floats2bfloat162_rn(__uint_as_float(o[q * 8 + 2 * i]) * inv_l, __uint_as_float(o[q * 8 + 2 * i + 1]) * inv_l);
          *reinterpret_cast<uint4*>(stage_row + (((c * 4 + q) ^ (lane & 7)) << 4)) = ov;
        }
      }
      __syncwarp();
      {
        const unsigned long long dst_u = reinterpret_cast<unsigned long long>(orow);
        const int row_ok = q_row < Sq;
#pragma unroll 4
        for (int it = 0; it < 16; ++it) {
          const int r_src = it * 2 + (lane >> 4), chunk = lane & 15;
          const unsigned long long d = __shfl_sync(0xffffffffu, dst_u, r_src);
          const int ok_row = __shfl_sync(0xffffffffu, row_ok, r_src);
          const uint4 v = *reinterpret_cast<const uint4*>(stage_warp + r_src * 256 + ((chunk ^ (r_src & 7)) << 4));
          if (ok_row) *reinterpret_cast<uint4*>(d + chunk * 16) = v;
        }
      }
      if (q_row < Sq) LSE[((size_t)b * H + h) * Sq + out_row] = (m_ref + log2f(l)) * 0.6931471805599453f;
    } else if (lane == 0) {
      atomicCAS(err, 0, 13);
      *abort_flag = 1;
    }
  } else {
    if (REGS) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(Sh::kRegsOther));   // the two padding warps of the third warpgroup
  }

  __syncwarp();
  if (*abort_flag) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Sh::kTmemCols);
  }
}

}  // namespace cb200

using namespace cb200;

template <int QT, int EXPM, int SPLITP, bool NA = false, bool REGS = false>
static int launch_fa_fwd(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, void* o, float* lse, int B, int Sq,
                         int Skv, int H, float scale, const SeqScatter& sc, int* err, cudaStream_t st,
                         const NaParams& na = NaParams{}) {
  using namespace fa;
  using Sh = Shape<QT, REGS>;
  auto kern = fa_fwd_kernel<QT, EXPM, SPLITP, NA, REGS>;
  static bool attr = false;
  if (!attr) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Sh::kSmem);
    if (e != cudaSuccess) return 100 + (int)e;
    if (REGS) {   // the register re-division inside the kernel is computed for exactly this launch allocation
      cudaFuncAttributes fa{};
      e = cudaFuncGetAttributes(&fa, kern);
      if (e != cudaSuccess) return 100 + (int)e;
      if (fa.numRegs != Sh::kRegsLaunch) return -43;
    }
    attr = true;
  }
  dim3 grid((Sq + QT * BQ - 1) / (QT * BQ), H, B);
  kern<<<grid, Sh::kThreads, Sh::kSmem, st>>>(tq, tk, tv, (bf16*)o, lse, Sq, Skv, H, scale * 1.4426950408889634f, sc, na, err);
  return (int)cudaGetLastError();
}

// the variant the operators use: exponentials split between the special-function unit and the FMA pipe, half-row hand-off
constexpr int kDefaultExpm = 1;     // one pair in four on the FMA pipe
constexpr int kDefaultSplit = 2;    // probabilities published in two halves
constexpr int kShortKeys = 1024;   // at most this many keys: the one-tile shape with two CTAs per SM

// q [B, Sq, H, 128]; k, v [B, Skv, H, 128]; o like q; lse [B, H, Sq] fp32.
// variant: 0 = default; 1..: tuning variants (all produce the same result within rounding)
static int fa_fwd_dispatch(const void* q, const void* k, const void* v, void* o, float* lse, int B, int Sq, int Skv, int H,
                           float scale, int variant, const SeqScatter& sc, int* err, cudaStream_t st,
                           const NaParams* na = nullptr) {
  using namespace fa;
  CUtensorMap tq, tk, tv;
  auto make = [&](CUtensorMap* m, const void* p, int S) {
    const uint64_t dims[4] = {(uint64_t)HD, (uint64_t)H, (uint64_t)S, (uint64_t)B};
    const uint64_t strides[3] = {(uint64_t)HD * 2, (uint64_t)H * HD * 2, (uint64_t)S * H * HD * 2};
    const uint32_t box[4] = {64, 1, 128, 1};
    return make_tmap_bf16(m, p, 4, dims, strides, box);
  };
  auto make_grid = [&](CUtensorMap* m, const void* p) {   // [B*T, Hg, Wg, heads, 128] seen through 4 x 4 x 8 token boxes
    const uint64_t Wg = (uint64_t)na->nW * 8, Hg = (uint64_t)na->nH * 4, Tg = (uint64_t)na->nT * 4;
    const uint64_t dims[5] = {(uint64_t)HD, (uint64_t)H, Wg, Hg, (uint64_t)B * Tg};
    const uint64_t strides[4] = {(uint64_t)HD * 2, (uint64_t)H * HD * 2, Wg * H * HD * 2, Hg * Wg * H * HD * 2};
    const uint32_t box[5] = {64, 1, 8, 4, 4};
    return make_tmap_bf16(m, p, 5, dims, strides, box);
  };
  int rc = na != nullptr ? make_grid(&tq, q) : make(&tq, q, Sq);
  if (rc) return rc;
  rc = na != nullptr ? make_grid(&tk, k) : make(&tk, k, Skv);
  if (rc) return rc;
  rc = na != nullptr ? make_grid(&tv, v) : make(&tv, v, Skv);
  if (rc) return rc;
  if (na != nullptr) return launch_fa_fwd<2, kDefaultExpm, kDefaultSplit, true, true>(tq, tk, tv, o, lse, B, Sq, Skv, H, scale, sc, err, st, *na);
  switch (variant) {
    case 1: return launch_fa_fwd<2, 0, 1>(tq, tk, tv, o, lse, B, Sq, Skv, H, scale, sc, err, st);   // all ex2, whole-row hand-off
    case 2: return launch_fa_fwd<2, 1, 2>(tq, tk, tv, o, lse, B, Sq, Skv, H, scale, sc, err, st);
    case 3: return launch_fa_fwd<2, 1, 1, false, true>(tq, tk, tv, o, lse, B, Sq, Skv, H, scale, sc, err, st);   // from here: register re-division, two issuers
    case 4: return launch_fa_fwd<2, 1, 2, false, true>(tq, tk, tv, o, lse, B, Sq, Skv, H, scale, sc, err, st);
    case 5: return launch_fa_fwd<2, 1, 4, false, true>(tq, tk, tv, o, lse, B, Sq, Skv, H, scale, sc, err, st);
    case 6: return launch_fa_fwd<2, 0, 2, false, true>(tq, tk, tv, o, lse, B, Sq, Skv, H, scale, sc, err, st);
    case 7: return launch_fa_fwd<1, kDefaultExpm, kDefaultSplit>(tq, tk, tv, o, lse, B, Sq, Skv, H, scale, sc, err, st);  // one tile, 2 CTAs / SM
    case 8: return launch_fa_fwd<1, 0, 1>(tq, tk, tv, o, lse, B, Sq, Skv, H, scale, sc, err, st);
    case 9: return launch_fa_fwd<2, 2, 2, false, true>(tq, tk, tv, o, lse, B, Sq, Skv, H, scale, sc, err, st);
    case 10: return launch_fa_fwd<2, 2, 4, false, true>(tq, tk, tv, o, lse, B, Sq, Skv, H, scale, sc, err, st);
    case 11: return launch_fa_fwd<2, 0, 4, false, true>(tq, tk, tv, o, lse, B, Sq, Skv, H, scale, sc, err, st);
    default: break;
  }
  if (sc.P == 0 && Skv <= kShortKeys) return launch_fa_fwd<1, kDefaultExpm, kDefaultSplit>(tq, tk, tv, o, lse, B, Sq, Skv, H, scale, sc, err, st);
  return launch_fa_fwd<2, kDefaultExpm, kDefaultSplit, false, true>(tq, tk, tv, o, lse, B, Sq, Skv, H, scale, sc, err, st);
}

extern "C" int cb200_fa_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int B, int Sq, int Skv, int H,
                            float scale, int variant, int* err, cudaStream_t st) {
  SeqScatter sc{};
  return fa_fwd_dispatch(q, k, v, o, lse, B, Sq, Skv, H, scale, variant, sc, err, st);
}

// Attention whose output rows are scattered to the P ranks' sequence shards (out_ptrs[r]: [B, Sq / P, P*H, 128] bf16 on rank r).
extern "C" int cb200_fa_fwd_scatter_seq(const void* q, const void* k, const void* v, const int64_t* out_ptrs, int P, int rank,
                                        float* lse, int B, int Sq, int Skv, int H, float scale, int* err, cudaStream_t st) {
  if (P < 1 || P > 8 || Sq % P != 0 || rank < 0 || rank >= P) return -21;
  SeqScatter sc{};
  for (int i = 0; i < P; ++i) sc.ptrs[i] = out_ptrs[i];
  sc.P = P;
  sc.rank = rank;
  sc.S_loc = Sq / P;
  return fa_fwd_dispatch(q, k, v, nullptr, lse, B, Sq, Skv, H, scale, 0, sc, err, st);
}

// Neighbourhood attention on a T x H x W token grid in natural order (see NaParams): self-attention, S = nT * nH * nW * 128.
extern "C" int cb200_fa_fwd_na(const void* q, const void* k, const void* v, void* o, float* lse, int B, int S, int H, float scale,
                               const int* kv_idx, const int* kv_cnt, int max_n, const uint8_t* bt, const uint8_t* bh,
                               const uint8_t* bw, int nT, int nH, int nW, int* err, cudaStream_t st) {
  if (nT < 1 || nH < 1 || nW < 1 || (long long)nT * nH * nW * 128 != (long long)S || max_n < 1) return -31;
  NaParams na{kv_idx, kv_cnt, bt, bh, bw, max_n, nT, nH, nW};
  SeqScatter sc{};
  return fa_fwd_dispatch(q, k, v, o, lse, B, S, S, H, scale, 0, sc, err, st, &na);
}
