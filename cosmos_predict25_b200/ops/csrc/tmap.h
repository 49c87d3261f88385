// Host-side construction of TMA tensor maps (driver entry point resolved at run time, so the
// extension does not link against libcuda).
#pragma once
#include <cuda.h>
#include <stdint.h>

namespace cb200 {

// rank-N bf16 tensor map with 128-byte swizzle. dims/box innermost first; strides_bytes has rank-1
// entries (stride of dims 1..rank-1). Returns 0 on success, a positive error code otherwise.
int make_tmap_bf16(CUtensorMap* out, const void* base, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
                   const uint32_t* box, int swizzle_128 = 1);

inline int make_tmap_2d_bf16(CUtensorMap* out, const void* base, uint64_t dim0, uint64_t dim1, uint64_t stride1_bytes,
                             uint32_t box0, uint32_t box1) {
  const uint64_t dims[2] = {dim0, dim1};
  const uint64_t strides[1] = {stride1_bytes};
  const uint32_t box[2] = {box0, box1};
  return make_tmap_bf16(out, base, 2, dims, strides, box);
}

}  // namespace cb200
