// Allocation-free entry point for callers that must not (or cannot) allocate device memory at call time.
//
// This entry point has no counterpart in the reference; it exists only in this library.
//
// Who needs it: code that is called from somebody else's runtime and has to obey that runtime's rules -
// an inference-server backend or plug-in whose execute/enqueue callback may not call cudaMalloc, a process
// that handed every byte of device memory to its own pool at start-up (so a later cudaMalloc simply fails),
// or a latency-critical loop that cannot afford the device-wide synchronisation an allocation implies. Such
// callers own their input and output buffers already; what they cannot provide is the scratch space the
// regular operator obtains from the framework allocator on every call.
//
// What it does: the backward pass of the per-head RMSNorm (+ optional rotate-half RoPE) operator - the same
// kernels as torch.ops.cosmos_b200.rmsnorm_rope_bwd - with the per-CTA partial sums of the weight gradient kept
// in a fixed array that lives inside the library image instead of in a freshly allocated tensor.
//
//   dy, x, dx : bf16 [n_rows, HD]  (n_rows = batch * tokens * heads, HD = 64 or 128)
//   w         : fp32 [HD]           rstd : fp32 [n_rows] (saved by the forward)
//   cosv,sinv : fp32 [S, HD/2] or both NULL when the forward applied no RoPE
//   dw        : fp32 [HD]           (output)
//
// Limits and rules
//   * n_rows <= CB200_NOALLOC_MAX_ROWS. Larger problems are rejected with CB200_NOALLOC_ERR_TOO_LARGE and a
//     message in errbuf; nothing is launched.
//   * The scratch array (CB200_NOALLOC_SCRATCH_FLOATS floats = 4 MiB) is part of the loaded library: every GPU on
//     which the library is used holds it until the process exits.
//   * The first call on each device looks up the array's device address (once per device, with that device
//     current). Make that first call during start-up, outside of any stream capture; later calls only launch.
//   * All calls on a device share the one array and it keeps whatever the previous call left in it. Each call
//     overwrites every slot it later reads, so nothing has to be cleared between calls; but two calls that
//     overlap on the GPU (different streams, no ordering between them) race on it. Serialise them.
//   * `stream` must be a stream of the device that is current when the call is made (or 0): the scratch address used is
//     the current device's, and a stream of another device would run the kernels against the wrong GPU's copy.
//   * No cudaMalloc / cudaFree / allocating library routine is called, on any path.
//
// Returns 0 on success, a negative CB200_NOALLOC_ERR_* code otherwise. errbuf (may be NULL) receives a
// human-readable reason of at most errbuf_len - 1 characters.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>

#define CB200_NOALLOC_SCRATCH_FLOATS (1u << 20)
#define CB200_NOALLOC_ROWS_PER_CTA 512            /* 8 warps x 64 rows */
#define CB200_NOALLOC_MAX_ROWS (4194304L)          /* (SCRATCH_FLOATS / 128) CTAs x 512 rows */

#define CB200_NOALLOC_ERR_TOO_LARGE (-1)
#define CB200_NOALLOC_ERR_BAD_ARGUMENT (-2)
#define CB200_NOALLOC_ERR_CUDA (-3)

#ifdef __cplusplus
extern "C" {
#endif

int cb200_rmsnorm_rope_bwd_noalloc(const void* dy, const void* x, const float* w, const float* rstd, const float* cosv,
                                   const float* sinv, void* dx, float* dw, long n_rows, int S, int H, int HD,
                                   cudaStream_t stream, char* errbuf, size_t errbuf_len);

#ifdef __cplusplus
}
#endif
