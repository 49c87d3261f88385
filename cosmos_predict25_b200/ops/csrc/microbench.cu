// Micro-benchmarks of hardware rates that bound the fused kernels (used by ops/bench_kernels.py only).
//
// red_f32: every warp adds 128-byte lines into an fp32 matrix with red.global.add.f32, with the access pattern of the
// single-pass attention backward (a CTA walks all rows of the matrix, many CTAs add into the same rows): measures the
// L2 reduction throughput that bounds the dQ accumulation.

#include <cuda_runtime.h>

#include "launchers.h"

namespace cb200 {

__global__ void __launch_bounds__(256) red_f32_bench_kernel(float* __restrict__ acc, int rows, int cols, int row_start_stride) {
  // CTA c starts at a different row so that concurrent CTAs mostly touch different rows at any instant, as in the real kernel
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int col0 = (warp & 3) * 32 + lane;                 // 4 warps cover 128 columns; the other 4 take the next row
  const int r0 = (int)(((long)blockIdx.x * row_start_stride) % rows);
  for (int r = (warp >> 2); r < rows; r += 2) {
    int rr = r0 + r;
    if (rr >= rows) rr -= rows;
    float* p = acc + (size_t)rr * cols + col0;
    asm volatile("red.global.add.f32 [%0], %1;" ::"l"(p), "f"(1.0f) : "memory");
  }
}

}  // namespace cb200

// adds 1.0 to every element of acc[rows, 128] from each of n_ctas CTAs: n_ctas * rows * 512 bytes of reductions
extern "C" int cb200_red_f32_bench(float* acc, int rows, int n_ctas, cudaStream_t st) {
  cb200::red_f32_bench_kernel<<<n_ctas, 256, 0, st>>>(acc, rows, 128, 977);
  return (int)cudaGetLastError();
}
