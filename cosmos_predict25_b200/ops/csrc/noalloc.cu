// Implementation of the allocation-free RMSNorm/RoPE backward entry point declared in noalloc.h.
//
// The scratch that the regular operator takes from the framework allocator is the file-scope device array
// below. Host code cannot use the array's name as a device pointer (on the host the name only stands for the
// symbol): the address a kernel can use is obtained once per device with cudaGetSymbolAddress, while that
// device is current, and cached. The kernels themselves are the ones behind torch.ops.cosmos_b200.rmsnorm_rope_bwd;
// they receive the cached address where they would otherwise receive a freshly allocated tensor.

#include "noalloc.h"

#include <stdio.h>

#include <mutex>

#include "launchers.h"

// per-CTA partial sums of the weight gradient: [n_ctas, HD]; part of the library image on every device
static __device__ __align__(256) float g_noalloc_scratch[CB200_NOALLOC_SCRATCH_FLOATS];

namespace {

constexpr int kMaxDevices = 64;
constexpr int kRowsPerWarp = CB200_RMSNORM_BWD_ROWS_PER_WARP;  // shared with the torch operator: same grouping, same bits
static_assert(CB200_NOALLOC_ROWS_PER_CTA == 8 * kRowsPerWarp, "noalloc.h states the rows per CTA of the backward kernel (8 warps)");
static_assert(CB200_NOALLOC_MAX_ROWS == (long)(CB200_NOALLOC_SCRATCH_FLOATS / 128) * CB200_NOALLOC_ROWS_PER_CTA,
              "the row limit follows from the scratch size at head_dim 128");

float* g_scratch_addr[kMaxDevices] = {nullptr};
std::mutex g_setup_mutex;

void set_error(char* errbuf, size_t n, const char* fmt, long a = 0, long b = 0) {
  if (errbuf != nullptr && n > 0) snprintf(errbuf, n, fmt, a, b);
}

// Device address of the scratch array for the current device (looked up on the first call per device).
cudaError_t scratch_for_current_device(float** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_scratch_addr[dev] == nullptr) {
    float* p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_noalloc_scratch);
    if (e != cudaSuccess) return e;
    g_scratch_addr[dev] = p;
  }
  *out = g_scratch_addr[dev];
  return cudaSuccess;
}

}  // namespace

extern "C" int cb200_rmsnorm_rope_bwd_noalloc(const void* dy, const void* x, const float* w, const float* rstd, const float* cosv,
                                              const float* sinv, void* dx, float* dw, long n_rows, int S, int H, int HD,
                                              cudaStream_t stream, char* errbuf, size_t errbuf_len) {
  if (dy == nullptr || x == nullptr || w == nullptr || rstd == nullptr || dx == nullptr || dw == nullptr) {
    set_error(errbuf, errbuf_len, "rmsnorm_rope_bwd_noalloc: a required pointer is NULL");
    return CB200_NOALLOC_ERR_BAD_ARGUMENT;
  }
  if ((HD != 64 && HD != 128) || n_rows <= 0 || S <= 0 || H <= 0 || (cosv == nullptr) != (sinv == nullptr)) {
    set_error(errbuf, errbuf_len, "rmsnorm_rope_bwd_noalloc: head_dim must be 64 or 128, sizes positive, cos/sin both set or both NULL");
    return CB200_NOALLOC_ERR_BAD_ARGUMENT;
  }
  const long ctas = cb200_rmsnorm_bwd_blocks(n_rows, kRowsPerWarp);
  if (n_rows > CB200_NOALLOC_MAX_ROWS || ctas * HD > (long)CB200_NOALLOC_SCRATCH_FLOATS) {
    set_error(errbuf, errbuf_len,
              "rmsnorm_rope_bwd_noalloc: %ld rows exceed the built-in scratch (at most %ld rows); use the allocating operator",
              n_rows, (long)CB200_NOALLOC_MAX_ROWS);
    return CB200_NOALLOC_ERR_TOO_LARGE;
  }
  float* scratch = nullptr;
  cudaError_t e = scratch_for_current_device(&scratch);
  if (e != cudaSuccess) {
    set_error(errbuf, errbuf_len, "rmsnorm_rope_bwd_noalloc: cudaGetSymbolAddress failed with CUDA error %ld", (long)e);
    return CB200_NOALLOC_ERR_CUDA;
  }
  // An error left behind by earlier, unrelated work must not be reported (and cleared) as this call's launch failure.
  e = cudaPeekAtLastError();
  if (e != cudaSuccess) {
    set_error(errbuf, errbuf_len, "rmsnorm_rope_bwd_noalloc: the CUDA context already carries error %ld from earlier work; nothing launched",
              (long)e);
    return CB200_NOALLOC_ERR_CUDA;
  }
  // every partial slot [0, ctas) x [0, HD) is written by the first kernel before the second one sums it
  cb200_rmsnorm_rope_bwd(dy, x, w, rstd, cosv, sinv, dx, dw, scratch, n_rows, S, H, HD, kRowsPerWarp, stream);
  e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error(errbuf, errbuf_len, "rmsnorm_rope_bwd_noalloc: kernel launch failed with CUDA error %ld", (long)e);
    return CB200_NOALLOC_ERR_CUDA;
  }
  return 0;
}
