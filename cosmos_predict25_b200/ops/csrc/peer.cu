// Kernels that fuse a collective with its neighbouring compute by loading from / storing to peer GPUs'
// memory over NVLink (plain ld/st through peer-mapped virtual addresses; no TMA, no multimem).
//
//   peer_barrier            signal every peer's flag word, then wait (bounded) for every peer's signal
//   rs_cast_norm_peer       FSDP reduce-scatter fused with bf16->fp32 cast, 1/world scale, NaN/Inf scrub
//                           and squared-norm partials: each rank READS its chunk of every peer's flat
//                           gradient buffer and sums in fp32
//   adamw_push_peer         sharded AdamW (+EMA) whose bf16 write-back is the all-gather: each updated
//                           chunk is STORED into every peer's full parameter buffer
//   a2a_scatter_heads_peer  Ulysses seq->head exchange: each 16-byte vector goes straight to the rank
//                           that owns its head (optionally after per-head RMSNorm + RoPE, so the q/k
//                           epilogue chain and the all-to-all are one kernel)
//   a2a_gather_seq_peer     Ulysses head->seq exchange (pull form): each rank reads its tokens of every
//                           peer's attention output
//
// Waits on remote flags are bounded: after kPeerSpinLimit probes the kernel writes an error code to
// `err` and returns, leaving the context usable.

#include "common.cuh"
#include "launchers.h"

namespace cb200 {

constexpr int kMaxPeers = 8;
constexpr unsigned kPeerSpinLimit = 1u << 24;  // default bound when the caller passes 0: ~1 us per probe => tens of seconds

struct PeerPtrs {
  void* p[kMaxPeers];
};

__device__ __forceinline__ void st_release_sys(unsigned* addr, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* addr) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}

// flags: per rank a symmetric array of kMaxPeers words; flags[r] on rank q is written by rank r.
// Thread p < P: publish `epoch` into peer p's slot [rank], then wait for our slot [p] to reach it.
__global__ void peer_barrier_kernel(PeerPtrs flags, int rank, int P, unsigned epoch, unsigned max_spins, int* err) {
  const int p = threadIdx.x;
  if (p < P) {
    __threadfence_system();
    st_release_sys(reinterpret_cast<unsigned*>(flags.p[p]) + rank, epoch);
    const unsigned* mine = reinterpret_cast<const unsigned*>(flags.p[rank]) + p;
    unsigned i = 0;
    // epochs grow monotonically; signed distance tolerates wrap-around
    while ((int)(ld_acquire_sys(mine) - epoch) < 0) {
      __nanosleep(100);
      if (++i >= max_spins) {
        atomicCAS(err, 0, 100 + p);
        break;
      }
    }
  }
}

// ---- reduce-scatter + cast + norm ---------------------------------------------------------------
struct Segment {
  long full_offset;   // element offset of the parameter in the full-layout buffer
  long stride;        // elements between consecutive ranks' chunks
  long shard_offset;  // element offset of the chunk in the shard-layout buffer
  long numel;         // chunk elements (multiple of 8)
};

__global__ void __launch_bounds__(256) rs_cast_norm_peer_kernel(PeerPtrs grads, const Segment* __restrict__ segs,
                                                                 float* __restrict__ g32, float* __restrict__ partials,
                                                                 int rank, int P, float scale) {
  __shared__ float red[32];
  const Segment sg = segs[blockIdx.y];
  const long nvec = sg.numel >> 3;
  const long src0 = sg.full_offset + (long)rank * sg.stride;
  float ss = 0.f;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long)gridDim.x * blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll 1
    for (int q = 0; q < P; ++q) {
      const int r = (rank + q) % P;  // start with the local copy, spread the remote reads over peers
      const bf16x8 v = *reinterpret_cast<const bf16x8*>(reinterpret_cast<const bf16*>(grads.p[r]) + src0 + i * 8);
      float f[8];
      unpack8(v, f);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += f[j];
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      acc[j] = scrub(acc[j] * scale);
      ss += acc[j] * acc[j];
    }
    float* dst = g32 + sg.shard_offset + i * 8;
    *reinterpret_cast<float4*>(dst) = make_float4(acc[0], acc[1], acc[2], acc[3]);
    *reinterpret_cast<float4*>(dst + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
  }
  const float t = block_sum(ss, red);
  if (threadIdx.x == 0) partials[blockIdx.y * gridDim.x + blockIdx.x] = t;
}

// unit_sumsq = sum(partials); total_sumsq += unit_sumsq  (single block => fixed summation order)
__global__ void finish_sumsq_kernel(const float* __restrict__ partials, int n, float* __restrict__ unit_sumsq,
                                    float* __restrict__ total_sumsq) {
  __shared__ float red[32];
  float s = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) s += partials[i];
  s = block_sum(s, red);
  if (threadIdx.x == 0) {
    unit_sumsq[0] = s;
    if (total_sumsq != nullptr) total_sumsq[0] += s;
  }
}

// ---- AdamW + EMA + all-gather by peer stores ---------------------------------------------------------
__global__ void __launch_bounds__(256) adamw_push_peer_kernel(
    PeerPtrs fulls, PeerPtrs sumsq_slots, const Segment* __restrict__ segs, float* __restrict__ master,
    const float* __restrict__ grad, float* __restrict__ m, float* __restrict__ v, float* __restrict__ ema, int rank, int P,
    float max_norm, float lr, float beta1, float beta2, float eps, float wd, float bc1, float rsqrt_bc2, float ema_beta,
    float* __restrict__ norm_out) {
  // global gradient norm from every rank's published squared sum (read over NVLink, 4 bytes per peer)
  float total = 0.f;
  for (int r = 0; r < P; ++r) total += *reinterpret_cast<const volatile float*>(sumsq_slots.p[r]);
  const float norm = sqrtf(total);
  const float clip = (max_norm > 0.f) ? fminf(max_norm / (norm + 1e-6f), 1.f) : 1.f;
  if (norm_out != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) norm_out[0] = norm;
  const Segment sg = segs[blockIdx.y];
  const long nvec = sg.numel >> 3;
  const long dst0 = sg.full_offset + (long)rank * sg.stride;
  const float decay = 1.f - lr * wd, step_size = lr / bc1, omb1 = 1.f - beta1, omb2 = 1.f - beta2;
  const bool do_ema = ema != nullptr && ema_beta >= 0.f;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long)gridDim.x * blockDim.x) {
    const long s0 = sg.shard_offset + i * 8;     // a multiple of 4 elements: 16-byte vector accesses throughout
    float gq[8], pq[8], mq[8], vq[8], eq[8];
    auto ld8 = [&](const float* src, float (&dst)[8]) {
      const float4 a = *reinterpret_cast<const float4*>(src + s0), b = *reinterpret_cast<const float4*>(src + s0 + 4);
      dst[0] = a.x; dst[1] = a.y; dst[2] = a.z; dst[3] = a.w; dst[4] = b.x; dst[5] = b.y; dst[6] = b.z; dst[7] = b.w;
    };
    auto st8 = [&](float* dst, const float (&src)[8]) {
      *reinterpret_cast<float4*>(dst + s0) = make_float4(src[0], src[1], src[2], src[3]);
      *reinterpret_cast<float4*>(dst + s0 + 4) = make_float4(src[4], src[5], src[6], src[7]);
    };
    ld8(grad, gq);
    ld8(master, pq);
    ld8(m, mq);
    ld8(v, vq);
    if (do_ema) ld8(ema, eq);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float g = gq[j] * clip;
      float p = pq[j] * decay;
      const float mi = beta1 * mq[j] + omb1 * g;
      const float vi = beta2 * vq[j] + omb2 * g * g;
      p -= step_size * (mi / (sqrtf(vi) * rsqrt_bc2 + eps));
      pq[j] = p;
      mq[j] = mi;
      vq[j] = vi;
      if (do_ema) eq[j] = ema_beta * eq[j] + (1.f - ema_beta) * p;
    }
    st8(master, pq);
    st8(m, mq);
    st8(v, vq);
    if (do_ema) st8(ema, eq);
    const bf16x8 packed = pack8(pq);
#pragma unroll 1
    for (int q = 0; q < P; ++q) {
      const int r = (rank + q) % P;
      *reinterpret_cast<bf16x8*>(reinterpret_cast<bf16*>(fulls.p[r]) + dst0 + i * 8) = packed;
    }
  }
}

// ---- Ulysses exchanges --------------------------------------------------------------------------------
// x [B, S, H, HD] local (all heads, local tokens) -> on rank p: out_p [B, P*S, H/P, HD], rows
// [rank*S, rank*S + S) filled with heads [p*H/P, (p+1)*H/P). One warp per (b, s, h) row of HD values.
// NORM: apply per-head RMSNorm with weight w and optional rotate-half RoPE first (cos/sin [S, HD/2]).
template <int HD, bool NORM>
__global__ void __launch_bounds__(256) a2a_scatter_heads_peer_kernel(
    const bf16* __restrict__ x, PeerPtrs outs, const float* __restrict__ w, const float* __restrict__ cosv,
    const float* __restrict__ sinv, float* __restrict__ rstd_out, long n_rows, int S, int H, int rank, int P, float eps) {
  constexpr int E = HD / 32;
  const int lane = threadIdx.x & 31;
  const long row = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= n_rows) return;
  const int hh = (int)(row % H);
  const long bs = row / H;
  const long s = bs % S;
  const long b = bs / S;
  const int Hl = H / P;
  const int dst_rank = hh / Hl;
  float v[E];
  const bf16* xr = x + row * HD + lane * E;
  if constexpr (E == 4) {
    const uint2 raw = *reinterpret_cast<const uint2*>(xr);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 c = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    v[0] = a.x; v[1] = a.y; v[2] = c.x; v[3] = c.y;
  } else {
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(xr));
    v[0] = a.x; v[1] = a.y;
  }
  if constexpr (NORM) {
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < E; ++j) ss += v[j] * v[j];
    ss = warp_sum(ss);
    const float rstd = rsqrtf(ss / HD + eps);
    if (lane == 0 && rstd_out != nullptr) rstd_out[row] = rstd;
#pragma unroll
    for (int j = 0; j < E; ++j) v[j] = v[j] * rstd * w[lane * E + j];
    if (cosv != nullptr) {
      const int half_idx = (lane & 15) * E;
#pragma unroll
      for (int j = 0; j < E; ++j) {
        const float other = __shfl_xor_sync(0xffffffffu, v[j], 16);
        const float c = cosv[s * (HD / 2) + half_idx + j];
        const float sn = sinv[s * (HD / 2) + half_idx + j];
        v[j] = (lane < 16) ? (v[j] * c - other * sn) : (v[j] * c + other * sn);
      }
    }
  }
  bf16* dst = reinterpret_cast<bf16*>(outs.p[dst_rank]) +
              (((b * P + rank) * (long)S + s) * Hl + (hh - dst_rank * Hl)) * HD + lane * E;
  if constexpr (E == 4) {
    uint2 raw;
    *reinterpret_cast<__nv_bfloat162*>(&raw.x) = __floats2bfloat162_rn(v[0], v[1]);
    *reinterpret_cast<__nv_bfloat162*>(&raw.y) = __floats2bfloat162_rn(v[2], v[3]);
    *reinterpret_cast<uint2*>(dst) = raw;
  } else {
    *reinterpret_cast<__nv_bfloat162*>(dst) = __floats2bfloat162_rn(v[0], v[1]);
  }
}

// o_p [B, P*S, Hl, HD] on every rank p (all tokens, local heads) -> out [B, S, H, HD] local: rank reads
// its token rows [rank*S, rank*S+S) from each peer p and places them at heads [p*Hl, (p+1)*Hl).
__global__ void __launch_bounds__(256) a2a_gather_seq_peer_kernel(PeerPtrs srcs, bf16* __restrict__ out, long nvec_total, int S,
                                                                   int H, int HD, int rank, int P) {
  const int Hl = H / P;
  const int vec_per_row = HD >> 3;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec_total; i += (long)gridDim.x * blockDim.x) {
    const int dv = (int)(i % vec_per_row);
    long t = i / vec_per_row;
    const int hh = (int)(t % H);
    t /= H;
    const long s = t % S;
    const long b = t / S;
    const int src_rank = hh / Hl;
    const bf16* src = reinterpret_cast<const bf16*>(srcs.p[src_rank]) +
                      (((b * P + rank) * (long)S + s) * Hl + (hh - src_rank * Hl)) * HD + dv * 8;
    reinterpret_cast<bf16x8*>(out)[i] = *reinterpret_cast<const bf16x8*>(src);
  }
}

// All-gather of small parameters by peer reads: for every segment (full_offset, rank_stride, shard_offset, numel) and every
// rank r, the chunk of `numel` bf16 values at shards[r] + shard_offset is copied to full + full_offset + r * rank_stride.
// grid = (blocks, segments, ranks); every count is a multiple of 8 elements (16-byte vectors).
__global__ void __launch_bounds__(256) gather_slots_peer_kernel(PeerPtrs shards, const Segment* __restrict__ segs, bf16* __restrict__ full) {
  const Segment sg = segs[blockIdx.y];
  const int r = blockIdx.z;
  const bf16x8* src = reinterpret_cast<const bf16x8*>(reinterpret_cast<const bf16*>(shards.p[r]) + sg.shard_offset);
  bf16x8* dst = reinterpret_cast<bf16x8*>(full + sg.full_offset + (long)r * sg.stride);
  const long nvec = sg.numel >> 3;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long)gridDim.x * blockDim.x) dst[i] = src[i];
}

}  // namespace cb200

using namespace cb200;

static PeerPtrs make_ptrs(const int64_t* ptrs, int P) {
  PeerPtrs pp;
  for (int i = 0; i < kMaxPeers; ++i) pp.p[i] = i < P ? reinterpret_cast<void*>(ptrs[i]) : nullptr;
  return pp;
}

extern "C" {

void cb200_peer_barrier(const int64_t* flag_ptrs, int rank, int P, unsigned epoch, unsigned max_spins, int* err, cudaStream_t st) {
  peer_barrier_kernel<<<1, 32, 0, st>>>(make_ptrs(flag_ptrs, P), rank, P, epoch, max_spins ? max_spins : kPeerSpinLimit, err);
}

int cb200_rs_blocks_x(void) { return 148 * 2; }

void cb200_rs_cast_norm_peer(const int64_t* grad_ptrs, const void* segs, int nseg, float* g32, float* partials, float* unit_sumsq,
                             float* total_sumsq, int rank, int P, float scale, cudaStream_t st) {
  dim3 grid(cb200_rs_blocks_x(), nseg);
  rs_cast_norm_peer_kernel<<<grid, 256, 0, st>>>(make_ptrs(grad_ptrs, P), (const Segment*)segs, g32, partials, rank, P, scale);
  finish_sumsq_kernel<<<1, 256, 0, st>>>(partials, cb200_rs_blocks_x() * nseg, unit_sumsq, total_sumsq);
}

void cb200_adamw_push_peer(const int64_t* full_ptrs, const int64_t* sumsq_ptrs, const void* segs, int nseg, float* master,
                           const float* grad, float* m, float* v, float* ema, int rank, int P, float max_norm, float lr,
                           float beta1, float beta2, float eps, float wd, long step, float ema_beta, float* norm_out,
                           cudaStream_t st) {
  const float bc1 = 1.f - powf(beta1, (float)step);
  const float bc2 = 1.f - powf(beta2, (float)step);
  dim3 grid(148 * 2, nseg);
  adamw_push_peer_kernel<<<grid, 256, 0, st>>>(make_ptrs(full_ptrs, P), make_ptrs(sumsq_ptrs, P), (const Segment*)segs, master,
                                               grad, m, v, ema, rank, P, max_norm, lr, beta1, beta2, eps, wd, bc1,
                                               1.f / sqrtf(bc2), ema_beta, norm_out);
}

void cb200_a2a_scatter_heads_peer(const void* x, const int64_t* out_ptrs, const float* w, const float* cosv, const float* sinv,
                                  float* rstd, long n_rows, int S, int H, int HD, int rank, int P, int norm, float eps,
                                  cudaStream_t st) {
  const unsigned blocks = (unsigned)((n_rows + 7) / 8);
  PeerPtrs pp = make_ptrs(out_ptrs, P);
#define LAUNCH(HDV, NV) \
  a2a_scatter_heads_peer_kernel<HDV, NV><<<blocks, 256, 0, st>>>((const bf16*)x, pp, w, cosv, sinv, rstd, n_rows, S, H, rank, P, eps)
  if (HD == 128) {
    if (norm) LAUNCH(128, true); else LAUNCH(128, false);
  } else {
    if (norm) LAUNCH(64, true); else LAUNCH(64, false);
  }
#undef LAUNCH
}

void cb200_gather_slots_peer(const int64_t* shard_ptrs, const void* segs, int nseg, void* full, int P, cudaStream_t st) {
  dim3 grid(8, nseg, P);
  gather_slots_peer_kernel<<<grid, 256, 0, st>>>(make_ptrs(shard_ptrs, P), (const Segment*)segs, (bf16*)full);
}

void cb200_a2a_gather_seq_peer(const int64_t* src_ptrs, void* out, long B, int S, int H, int HD, int rank, int P, cudaStream_t st) {
  const long nvec = B * S * H * (HD >> 3);
  long blocks = (nvec + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  a2a_gather_seq_peer_kernel<<<(unsigned)blocks, 256, 0, st>>>(make_ptrs(src_ptrs, P), (bf16*)out, nvec, S, H, HD, rank, P);
}

}  // extern "C"
