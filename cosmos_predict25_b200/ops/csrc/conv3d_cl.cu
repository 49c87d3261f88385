// Convolution on channels-last activations as an implicit GEMM on the 5th-generation tensor cores (sm_100a), bf16 in / fp32 accumulate.
//
// Serves every convolution of the Wan-style causal VAE decoder (cosmos_predict2/_src/predict2/tokenizers/wan2pt1.py:40-58 causal
// Conv3d, :84-137 resample, :184-215 residual block): 3 x 3 x 3 causal, 3 x 1 x 1 temporal, 3 x 3 spatial (as the four 2 x 2 phase
// convolutions of "nearest 2x up-sampling followed by 3 x 3"), 1 x 1 x 1.
//
//   activation X [T_in, H_in, W_in, C_in]   (C_in a multiple of 16)
//   weights    W [N_pad, taps, C_pad]        (K-major; C_pad = C_in rounded up to 64, N_pad = C_out rounded up to the N tile)
//   output     Y[t, h, w, n] = bias[n] + sum_{tap, c} X[t + dt(tap), h + dh(tap), w + dw(tap), c] * W[n, tap, c]  (+ residual)
//
// There is no im2col buffer: an output tile is 128 voxels = 8 rows x 16 columns of one frame, and the A operand of tap
// (dt, dh, dw), channel block kb is the TMA box {64 channels, 16 w, 8 h, 1 t} at coordinates (64 kb, w0 + dw, h0 + dh, t + dt) of
// the activation tensor itself. It lands in shared memory as a [128 rows][64 channels] 128-byte-swizzled K-major tile, which is
// what the MMA wants. Coordinates outside the tensor read zeros: that IS the zero padding of the convolution (the channel
// coordinate stays a multiple of 64, so the 16-byte alignment rule of TMA holds for every tap). The causal time padding is
// two leading frames of the input tensor (the stream cache of the previous chunk, or zeros).
//
// Persistent, warp-specialised, one CTA per SM, same skeleton as the GEMM of this package: warp 0 TMA producer (4-stage ring of
// A box + B box), warp 1 MMA issuer (UMMA 128 x N x 16 into one of two TMEM accumulators), warps 2-9 epilogue (bias, optional
// residual, bf16 store through a per-voxel output mapping that also expresses the phase interleave of the up-sampling
// convolutions and the frame interleave of the temporal up-sampler). All waits are bounded and report through `err`.

#include <math.h>

#include "common.cuh"
#include "launchers.h"
#include "sm100.cuh"
#include "tmap.h"

namespace cb200 {
using namespace sm100;

namespace cv {
constexpr int BM = 128, BK = 64, TH = 8, TW = 16;
constexpr int kStages = 4;
constexpr int kABytes = BM * BK * 2;          // 16 KB
constexpr int kBMaxBytes = 256 * BK * 2;      // 32 KB
constexpr int kStageBytes = kABytes + kBMaxBytes;
constexpr int kThreads = 320;                 // TMA warp, MMA warp, 8 epilogue warps
constexpr size_t kSmem = (size_t)kStages * kStageBytes + 1024 + 256;
constexpr int kMaxTaps = 27;
}  // namespace cv

struct ConvParams {
  int T_out, H_out, W_out;      // output grid walked by the tiles
  int Cin, Cout;
  int n_tile, tiles_n;          // N per tile (multiple of 16, <= 256) and number of N tiles
  int ntaps, kblocks;           // K loop: taps x 64-channel blocks
  int8_t dt[cv::kMaxTaps], dh[cv::kMaxTaps], dw[cv::kMaxTaps];   // input coordinate = output coordinate + offset
  // element offset of output voxel (t, h, w), channel n:
  //   (((t * ot_mul + ot_add) * out_H + h * oh_mul + oh_add) * out_W + w * ow_mul + ow_add) * out_C + oc_add + n
  int ot_mul, ot_add, oh_mul, oh_add, ow_mul, ow_add, out_H, out_W, out_C, oc_add;
  bf16* Y;
  const bf16* resid;            // optional, same addressing as Y
  const float* bias;            // optional [Cout]
};

__global__ void __launch_bounds__(cv::kThreads, 1)
conv_cl_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_w, const ConvParams p,
               int* __restrict__ err) {
  using namespace cv;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes);
  uint64_t* full = bars;                    // [kStages]
  uint64_t* empty = bars + kStages;         // [kStages]
  uint64_t* acc_full = bars + 2 * kStages;  // [2]
  uint64_t* acc_empty = acc_full + 2;       // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  // the shuffle makes the warp index (and every role branch below) provably warp-uniform for the compiler
  const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;
  const int tiles_w = (p.W_out + TW - 1) / TW, tiles_h = (p.H_out + TH - 1) / TH;
  const int n_tiles = p.T_out * tiles_h * tiles_w * p.tiles_n;
  const int b_bytes = p.n_tile * BK * 2;

  if (threadIdx.x == 0) *abort_flag = *reinterpret_cast<volatile int*>(err);   // an earlier error: drain the grid at once
  __syncthreads();
  if (*abort_flag != 0) return;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], 8);
    }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // tile index -> (n tile, w tile, h tile, frame); N tiles of one voxel tile are neighbours so that they run at the same time
  // on different SMs and share the activation boxes through L2
  auto decode = [&](int t, int& nt, int& w0, int& h0, int& tf) {
    nt = t % p.tiles_n;
    t /= p.tiles_n;
    w0 = (t % tiles_w) * TW;
    t /= tiles_w;
    h0 = (t % tiles_h) * TH;
    tf = t / tiles_h;
  };

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      prefetch_tmap(&tm_x);
      prefetch_tmap(&tm_w);
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x) {
        int nt, w0, h0, tf;
        decode(t, nt, w0, h0, tf);
        for (int tap = 0; tap < p.ntaps && ok; ++tap) {
          for (int kb = 0; kb < p.kblocks; ++kb) {
            if (!mbar_wait(&empty[s], ph ^ 1, abort_flag)) { ok = false; break; }
            uint8_t* sa = smem + s * kStageBytes;
            mbar_arrive_expect_tx(&full[s], kABytes + b_bytes);
            tma_load_4d(sa, &tm_x, &full[s], kb * BK, w0 + p.dw[tap], h0 + p.dh[tap], tf + p.dt[tap]);
            tma_load_2d(sa + kABytes, &tm_w, &full[s], (tap * p.kblocks + kb) * BK, nt * p.n_tile);
            if (++s == kStages) { s = 0; ph ^= 1; }
          }
        }
      }
      if (!ok) { atomicCAS(err, 0, 61); *abort_flag = 1; }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (warp-uniform; the elected lane issues)
    const uint32_t leader = elect_one() ? 1u : 0u;
    auto wait_all = [&](uint64_t* bar, uint32_t parity) -> bool { return __all_sync(0xffffffffu, mbar_wait(bar, parity, abort_flag)); };
    const uint32_t idesc = umma_idesc_bf16(BM, p.n_tile, 0, 0);
    const uint64_t da0 = umma_desc_sw128(smem_u32(smem), 16, 1024);
    const uint64_t db0 = umma_desc_sw128(smem_u32(smem) + kABytes, 16, 1024);
    int s = 0;
    uint32_t ph = 0;
    int acc = 0;
    uint32_t acc_ph = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x) {
      if (!wait_all(&acc_empty[acc], acc_ph ^ 1)) { ok = false; break; }
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + acc * 256;
      uint32_t first = 0;
      for (int tap = 0; tap < p.ntaps && ok; ++tap) {
        for (int kb = 0; kb < p.kblocks; ++kb) {
          if (!wait_all(&full[s], ph)) { ok = false; break; }
          tc_fence_after();
          const uint64_t da_s = da0 + (uint64_t)(s * (kStageBytes >> 4)), db_s = db0 + (uint64_t)(s * (kStageBytes >> 4));
          const int ksteps = min(4, (p.Cin - kb * BK) / 16);   // the last channel block of C_in = 96 holds 32 real channels
          for (int k = 0; k < ksteps; ++k) {
            umma_ss_w(d_tmem, da_s + (uint32_t)((k * 32) >> 4), db_s + (uint32_t)((k * 32) >> 4), idesc, first, leader);
            first = 1u;
          }
          umma_commit_w(&empty[s], leader);  // slot reusable once these MMAs have read it
          if (++s == kStages) { s = 0; ph ^= 1; }
        }
      }
      if (!ok) break;
      umma_commit_w(&acc_full[acc], leader);
      if (++acc == 2) { acc = 0; acc_ph ^= 1; }
    }
    if (!ok && lane == 0) { atomicCAS(err, 0, 62); *abort_flag = 1; }
  } else {
    // ------------------------------------------------------------------ epilogue warps: a thread owns one output voxel
    const int quarter = warp & 3;      // TMEM lanes [32 quarter, +32)
    const int part = (warp - 2) >> 2;  // which half of the tile's 16-column chunks
    const int r = quarter * 32 + lane; // row of the tile = (h, w) of the voxel inside the 8 x 16 patch
    const int hh = r >> 4, ww = r & 15;
    const int nch = p.n_tile >> 4, c_lo = part == 0 ? 0 : (nch + 1) / 2, c_hi = part == 0 ? (nch + 1) / 2 : nch;
    int acc = 0;
    uint32_t acc_ph = 0;
    bool ok = true;
    const bool vec_ok = ((p.out_C | p.oc_add) & 7) == 0;
    for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x) {
      int nt, w0, h0, tf;
      decode(t, nt, w0, h0, tf);
      if (!mbar_wait(&acc_full[acc], acc_ph, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const int h = h0 + hh, w = w0 + ww;
      const bool valid = h < p.H_out && w < p.W_out;
      const size_t vox = ((size_t)(tf * p.ot_mul + p.ot_add) * p.out_H + (h * p.oh_mul + p.oh_add)) * p.out_W + (w * p.ow_mul + p.ow_add);
      const size_t base = vox * p.out_C + p.oc_add;
      const uint32_t t_row = tmem_base + acc * 256 + ((uint32_t)(quarter * 32) << 16);
#pragma unroll 1
      for (int c = c_lo; c < c_hi; ++c) {
        uint32_t a[16];
        tmem_ld16(t_row + c * 16, a);      // warp-collective: every lane runs it, invalid voxels only skip their stores
        tmem_ld_wait();
        const int n0 = nt * p.n_tile + c * 16;
        if (valid && n0 < p.Cout) {
          float v[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = __uint_as_float(a[j]);
          const bool full_chunk = vec_ok && n0 + 16 <= p.Cout;
          if (p.bias != nullptr) {
#pragma unroll
            for (int j = 0; j < 16; ++j)
              if (full_chunk || n0 + j < p.Cout) v[j] += p.bias[n0 + j];
          }
          if (full_chunk) {
            if (p.resid != nullptr) {
#pragma unroll
              for (int q = 0; q < 2; ++q) {
                const uint4 rr = *reinterpret_cast<const uint4*>(p.resid + base + n0 + q * 8);
                const __nv_bfloat162* r2 = reinterpret_cast<const __nv_bfloat162*>(&rr);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const float2 rf = __bfloat1622float2(r2[j]);
                  v[q * 8 + 2 * j] += rf.x;
                  v[q * 8 + 2 * j + 1] += rf.y;
                }
              }
            }
#pragma unroll
            for (int q = 0; q < 2; ++q) {
              uint4 o;
              __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
              for (int j = 0; j < 4; ++j) o2[j] = __floats2bfloat162_rn(v[q * 8 + 2 * j], v[q * 8 + 2 * j + 1]);
              *reinterpret_cast<uint4*>(p.Y + base + n0 + q * 8) = o;
            }
          } else {
            for (int j = 0; j < 16 && n0 + j < p.Cout; ++j) {
              float o = v[j];
              if (p.resid != nullptr) o += __bfloat162float(p.resid[base + n0 + j]);
              p.Y[base + n0 + j] = __float2bfloat16(o);
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[acc]);
      if (++acc == 2) { acc = 0; acc_ph ^= 1; }
    }
    if (!ok && lane == 0) { atomicCAS(err, 0, 63); *abort_flag = 1; }
  }

  __syncwarp();
  if (*abort_flag) {
    // let outstanding bulk copies / MMAs drain before shared memory and TMEM go away
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// y[v, :] = silu(x[v, :] / max(||x[v, :]||_2, 1e-12) * sqrt(C) * gamma): the RMS-norm + SiLU in front of every convolution of a
// residual block, on channels-last rows (one warp per voxel, 16-byte accesses; C a multiple of 8, at most 1024).
__global__ void __launch_bounds__(256) rmsnorm_silu_cl_kernel(const bf16* __restrict__ x, const float* __restrict__ gamma,
                                                                bf16* __restrict__ y, long n_vox, int C, float scale, int silu) {
  const int lane = threadIdx.x & 31;
  const long v = (long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (v >= n_vox) return;
  const bf16* row = x + v * C;
  bf16* out = y + v * C;
  const int nvec = C >> 3;
  float vals[4][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int idx = lane + i * 32;
    if (idx < nvec) {
      const bf16x8 pk = *reinterpret_cast<const bf16x8*>(row + idx * 8);
      unpack8(pk, vals[i]);
#pragma unroll
      for (int j = 0; j < 8; ++j) ss = fmaf(vals[i][j], vals[i][j], ss);
    }
  }
  ss = warp_sum(ss);
  const float inv = scale / fmaxf(sqrtf(ss), 1e-12f);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int idx = lane + i * 32;
    if (idx < nvec) {
      float o[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float z = vals[i][j] * inv * gamma[idx * 8 + j];
        o[j] = silu ? z / (1.f + __expf(-z)) : z;
      }
      *reinterpret_cast<bf16x8*>(out + idx * 8) = pack8(o);
    }
  }
}

}  // namespace cb200

using namespace cb200;

// x [T_in, H_in, W_in, Cin] bf16; w [n_rows, ntaps * kblocks * 64] bf16 with n_rows = tiles_n * n_tile; taps: ntaps x (dt, dh, dw).
// out_map: {ot_mul, ot_add, oh_mul, oh_add, ow_mul, ow_add, out_H, out_W, out_C, oc_add}.
extern "C" int cb200_conv_cl(const void* x, int T_in, int H_in, int W_in, int Cin, const void* w, int n_rows, int n_tile, int Cout,
                             const int* taps, int ntaps, int T_out, int H_out, int W_out, const int* out_map, void* y,
                             const void* resid, const float* bias, int* err, int sms, cudaStream_t st) {
  using namespace cv;
  if (Cin % 16 != 0 || Cin < 16 || ntaps < 1 || ntaps > kMaxTaps || n_tile % 16 != 0 || n_tile < 16 || n_tile > 256 ||
      n_rows % n_tile != 0 || Cout > n_rows || Cout < 1)
    return -51;
  ConvParams p{};
  p.T_out = T_out;
  p.H_out = H_out;
  p.W_out = W_out;
  p.Cin = Cin;
  p.Cout = Cout;
  p.n_tile = n_tile;
  p.tiles_n = (Cout + n_tile - 1) / n_tile;
  p.ntaps = ntaps;
  p.kblocks = (Cin + BK - 1) / BK;
  for (int i = 0; i < ntaps; ++i) {
    const int dt = taps[3 * i], dh = taps[3 * i + 1], dw = taps[3 * i + 2];
    if (dt < -64 || dt > 64 || dh < -64 || dh > 64 || dw < -64 || dw > 64) return -52;
    p.dt[i] = (int8_t)dt;
    p.dh[i] = (int8_t)dh;
    p.dw[i] = (int8_t)dw;
  }
  p.ot_mul = out_map[0];
  p.ot_add = out_map[1];
  p.oh_mul = out_map[2];
  p.oh_add = out_map[3];
  p.ow_mul = out_map[4];
  p.ow_add = out_map[5];
  p.out_H = out_map[6];
  p.out_W = out_map[7];
  p.out_C = out_map[8];
  p.oc_add = out_map[9];
  p.Y = (bf16*)y;
  p.resid = (const bf16*)resid;
  p.bias = bias;
  CUtensorMap tx, tw;
  {
    const uint64_t dims[4] = {(uint64_t)Cin, (uint64_t)W_in, (uint64_t)H_in, (uint64_t)T_in};
    const uint64_t strides[3] = {(uint64_t)Cin * 2, (uint64_t)W_in * Cin * 2, (uint64_t)H_in * W_in * Cin * 2};
    const uint32_t box[4] = {BK, TW, TH, 1};
    const int rc = make_tmap_bf16(&tx, x, 4, dims, strides, box);
    if (rc) return rc;
  }
  {
    const uint64_t kdim = (uint64_t)ntaps * p.kblocks * BK;
    const int rc = make_tmap_2d_bf16(&tw, w, kdim, (uint64_t)n_rows, kdim * 2, BK, (uint32_t)n_tile);
    if (rc) return rc;
  }
  static bool attr = false;
  if (!attr) {
    cudaError_t e = cudaFuncSetAttribute(conv_cl_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmem);
    if (e != cudaSuccess) return 100 + (int)e;
    attr = true;
  }
  const long tiles = (long)T_out * ((H_out + TH - 1) / TH) * ((W_out + TW - 1) / TW) * p.tiles_n;
  if (tiles <= 0 || tiles > 0x7fffffffL) return -53;
  const int grid = tiles < sms ? (int)tiles : sms;
  conv_cl_kernel<<<grid, kThreads, kSmem, st>>>(tx, tw, p, err);
  return (int)cudaGetLastError();
}

extern "C" int cb200_rmsnorm_silu_cl(const void* x, const float* gamma, void* y, long n_vox, int C, int silu, cudaStream_t st) {
  if (C % 8 != 0 || C > 1024 || n_vox <= 0) return -54;
  rmsnorm_silu_cl_kernel<<<(unsigned)((n_vox + 7) / 8), 256, 0, st>>>((const bf16*)x, gamma, (bf16*)y, n_vox, C, sqrtf((float)C), silu);
  return (int)cudaGetLastError();
}
