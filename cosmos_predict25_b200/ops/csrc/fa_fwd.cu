// Flash attention forward on tcgen05 / TMEM (sm_100a), head_dim 128, bf16, non-causal.
//
// One CTA owns two 128-row query tiles of one (batch, head) and walks over the keys in tiles of 128:
//
//   warps 0-3   softmax of query tile 0   (thread i <-> query row i <-> TMEM lane i)
//   warps 4-7   softmax of query tile 1
//   warp  8     TMA producer: Q once, then K_j and V_j through two 2-slot rings (128-byte swizzle)
//   warp  9     MMA issuer (one thread): S_t = Q_t K_j^T  (SS form, both operands K-major in smem)
//                                        O_t += P_t V_j   (TS form: P read from TMEM, V N-major in smem)
//
// TMEM (512 columns): S_0 [0,128) S_1 [128,256) fp32 scores, O_0 [256,384) O_1 [384,512) fp32 outputs.
// The softmax thread reads its score row with tcgen05.ld, and writes the bf16 probabilities back over
// the first 64 columns of the same S buffer with tcgen05.st; the P·V MMA takes them from there, so
// probabilities never visit shared memory. While one tile is in softmax the tensor core runs the
// other tile's P·V and next Q·K^T (ping-pong).
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
constexpr int kThreads = 320;
constexpr size_t kSmem = 6 * (size_t)kTileBytes + 1024 + 256;
constexpr float kRescaleThreshold = 8.0f;  // log2 units
}  // namespace fa

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__global__ void __launch_bounds__(fa::kThreads, 1)
fa_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
              const __grid_constant__ CUtensorMap tm_v, bf16* __restrict__ O, float* __restrict__ LSE, int Sq, int Skv, int H,
              float scale_log2, int* __restrict__ err) {
  using namespace fa;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = smem;                    // 2 tiles
  uint8_t* sK = smem + 2 * kTileBytes;   // 2 slots
  uint8_t* sV = smem + 4 * kTileBytes;   // 2 slots
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 6 * kTileBytes);
  uint64_t* q_full = bars;        // [1]
  uint64_t* k_full = bars + 1;    // [2]
  uint64_t* k_empty = bars + 3;   // [2]
  uint64_t* v_full = bars + 5;    // [2]
  uint64_t* v_empty = bars + 7;   // [2]
  uint64_t* s_full = bars + 9;    // [2]  scores of tile t ready (also: all earlier MMAs of the CTA complete)
  uint64_t* p_ready = bars + 11;  // [2]  probabilities of tile t written to TMEM
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 13);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.y, b = blockIdx.z;
  const int q_base = blockIdx.x * 2 * BQ;
  const int n_kv = (Skv + BKV - 1) / BKV;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&p_ready[i], 4);
    }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 9) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 8) {
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
      for (int j = 0; j < n_kv && ok; ++j) {
        const int slot = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(&k_empty[slot], ph ^ 1, abort_flag)) { ok = false; break; }
        mbar_arrive_expect_tx(&k_full[slot], kTileBytes);
        for (int c = 0; c < 2; ++c) tma_load_4d(sK + slot * kTileBytes + c * kHalfBytes, &tm_k, &k_full[slot], c * 64, h, j * BKV, b);
        if (!mbar_wait(&v_empty[slot], ph ^ 1, abort_flag)) { ok = false; break; }
        mbar_arrive_expect_tx(&v_full[slot], kTileBytes);
        for (int c = 0; c < 2; ++c) tma_load_4d(sV + slot * kTileBytes + c * kHalfBytes, &tm_v, &v_full[slot], c * 64, h, j * BKV, b);
      }
      if (!ok) { atomicCAS(err, 0, 11); *abort_flag = 1; }
    }
  } else if (warp == 9) {
    // -------------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_qk = umma_idesc_bf16(128, 128, 0, 0);
      constexpr uint32_t idesc_pv = umma_idesc_bf16(128, 128, 0, 1);
      bool ok = mbar_wait(q_full, 0, abort_flag);
      auto issue_qk = [&](int t, int slot) {
        const uint32_t qa = smem_u32(sQ + t * kTileBytes), ka = smem_u32(sK + slot * kTileBytes);
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t off = (kk >> 2) * kHalfBytes + (kk & 3) * 32;
          umma_ss(tmem_base + t * 128, umma_desc_sw128(qa + off, 16, 1024), umma_desc_sw128(ka + off, 16, 1024), idesc_qk,
                  kk > 0 ? 1u : 0u);
        }
      };
      auto issue_pv = [&](int t, int slot, bool accumulate) {
        const uint32_t va = smem_u32(sV + slot * kTileBytes);
#pragma unroll
        for (int kk = 0; kk < BKV / 16; ++kk) {
          umma_ts(tmem_base + 256 + t * 128, tmem_base + t * 128 + kk * 8, umma_desc_sw128(va + kk * 2048, kHalfBytes, 1024),
                  idesc_pv, (accumulate || kk > 0) ? 1u : 0u);
        }
      };
      if (ok) ok = mbar_wait(&k_full[0], 0, abort_flag);
      if (ok) {
        tc_fence_after();
        issue_qk(0, 0);
        umma_commit(&s_full[0]);
        issue_qk(1, 0);
        umma_commit(&s_full[1]);
        umma_commit(&k_empty[0]);
      }
      for (int j = 0; j < n_kv && ok; ++j) {
        const int slot = j & 1, nslot = (j + 1) & 1;
        const uint32_t ph = (j >> 1) & 1, nph = ((j + 1) >> 1) & 1;
        const bool has_next = (j + 1) < n_kv;
        if (!mbar_wait(&v_full[slot], ph, abort_flag)) { ok = false; break; }
        if (has_next && !mbar_wait(&k_full[nslot], nph, abort_flag)) { ok = false; break; }
        for (int t = 0; t < 2; ++t) {
          if (!mbar_wait(&p_ready[t], j & 1, abort_flag)) { ok = false; break; }
          tc_fence_after();
          issue_pv(t, slot, j > 0);
          if (t == 1) umma_commit(&v_empty[slot]);
          if (has_next) issue_qk(t, nslot);
          // K_{j+1} is free again once tile 1's Q.K^T on it has completed
          if (t == 1 && has_next) umma_commit(&k_empty[nslot]);
          umma_commit(&s_full[t]);
        }
      }
      if (!ok) { atomicCAS(err, 0, 12); *abort_flag = 1; }
    }
  } else {
    // -------------------------------------------------------------------- softmax warpgroups
    const int t = warp >> 2;       // query tile
    const int quarter = warp & 3;  // TMEM lane quarter
    const int q_row = q_base + t * BQ + quarter * 32 + lane;
    const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
    const uint32_t tS = tmem_base + t * 128 + lane_off;
    const uint32_t tO = tmem_base + 256 + t * 128 + lane_off;
    float m_ref = -INFINITY;  // reference maximum used in the exponent (log2 domain)
    float l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_kv; ++j) {
      if (!mbar_wait(&s_full[t], j & 1, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const int n_valid = min(BKV, Skv - j * BKV);
      // pass 1: row maximum
      float mx = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        tmem_ld32(tS + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const float s = __uint_as_float(r[i]);
          mx = fmaxf(mx, (c * 32 + i < n_valid) ? s : -INFINITY);
        }
      }
      mx *= scale_log2;
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
          uint32_t r[32];
          tmem_ld32(tO + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
          tmem_st32(tO + c * 32, r);
        }
        tmem_st_wait();
      }
      // pass 2: probabilities -> bf16 pairs over the first 64 columns of the score buffer
      float lsum = 0.f;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        tmem_ld32(tS + c * 32, r);
        tmem_ld_wait();
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float p0 = ex2(__uint_as_float(r[2 * i]) * scale_log2 - m_ref);
          float p1 = ex2(__uint_as_float(r[2 * i + 1]) * scale_log2 - m_ref);
          if (c * 32 + 2 * i >= n_valid) p0 = 0.f;
          if (c * 32 + 2 * i + 1 >= n_valid) p1 = 0.f;
          lsum += p0 + p1;
          __nv_bfloat162 pb = __floats2bfloat162_rn(p0, p1);
          pk[i] = *reinterpret_cast<uint32_t*>(&pb);
        }
        asm volatile(
            "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
            ::"r"(tS + c * 16), "r"(pk[0]), "r"(pk[1]), "r"(pk[2]), "r"(pk[3]), "r"(pk[4]), "r"(pk[5]), "r"(pk[6]), "r"(pk[7]),
              "r"(pk[8]), "r"(pk[9]), "r"(pk[10]), "r"(pk[11]), "r"(pk[12]), "r"(pk[13]), "r"(pk[14]), "r"(pk[15])
            : "memory");
      }
      l += lsum;
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_ready[t]);
    }
    if (ok) ok = mbar_wait(&s_full[t], n_kv & 1, abort_flag);
    if (ok) {
      tc_fence_after();
      const float inv_l = 1.f / l;
      bf16* orow = O + (((size_t)b * Sq + q_row) * H + h) * HD;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        tmem_ld32(tO + c * 32, r);
        tmem_ld_wait();
        if (q_row < Sq) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 o;
            __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
            for (int i = 0; i < 4; ++i)
              o2[i] = __floats2bfloat162_rn(__uint_as_float(r[q * 8 + 2 * i]) * inv_l, __uint_as_float(r[q * 8 + 2 * i + 1]) * inv_l);
            *reinterpret_cast<uint4*>(orow + c * 32 + q * 8) = o;
          }
        }
      }
      if (q_row < Sq) LSE[((size_t)b * H + h) * Sq + q_row] = (m_ref + log2f(l)) * 0.6931471805599453f;
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
  if (warp == 9) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace cb200

using namespace cb200;

// q [B, Sq, H, 128]; k, v [B, Skv, H, 128]; o like q; lse [B, H, Sq] fp32
extern "C" int cb200_fa_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int B, int Sq, int Skv, int H,
                            float scale, int* err, cudaStream_t st) {
  using namespace fa;
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
  static bool attr = false;
  if (!attr) {
    cudaError_t e = cudaFuncSetAttribute(fa_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmem);
    if (e != cudaSuccess) return 100 + (int)e;
    attr = true;
  }
  dim3 grid((Sq + 2 * BQ - 1) / (2 * BQ), H, B);
  fa_fwd_kernel<<<grid, kThreads, kSmem, st>>>(tq, tk, tv, (bf16*)o, lse, Sq, Skv, H, scale * 1.4426950408889634f, err);
  return (int)cudaGetLastError();
}
