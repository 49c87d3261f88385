#include "tmap.h"

#include <cuda_runtime.h>

#include <cstring>
#include <mutex>
#include <unordered_map>

namespace cb200 {

// A tensor map is a pure function of (address, shape, strides, box, swizzle): the training loop presents the same few hundred
// combinations every step (weights, activations at cached allocator addresses), so encoded maps are kept and looked up instead
// of calling the driver for every launch.
namespace {
struct TmapKey {
  uint64_t v[17];
  bool operator==(const TmapKey& o) const { return std::memcmp(v, o.v, sizeof(v)) == 0; }
};
struct TmapKeyHash {
  size_t operator()(const TmapKey& k) const {
    uint64_t h = 0xcbf29ce484222325ull;
    for (uint64_t x : k.v) h = (h ^ x) * 0x100000001b3ull;
    return (size_t)h;
  }
};
constexpr size_t kTmapCacheLimit = 16384;
std::mutex g_tmap_mu;
std::unordered_map<TmapKey, CUtensorMap, TmapKeyHash> g_tmap_cache;
}  // namespace

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn resolve_encode() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

int make_tmap_bf16(CUtensorMap* out, const void* base, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
                   const uint32_t* box, int swizzle_128) {
  EncodeTiledFn fn = resolve_encode();
  if (fn == nullptr) return 901;
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) return 902;
  if (rank < 1 || rank > 5) return 904;
  TmapKey key;
  std::memset(&key, 0, sizeof(key));
  key.v[0] = reinterpret_cast<uintptr_t>(base);
  key.v[1] = ((uint64_t)rank << 1) | (uint64_t)(swizzle_128 ? 1 : 0);
  for (int i = 0; i < rank; ++i) {
    key.v[2 + i] = dims[i];
    key.v[7 + i] = box[i];
    if (i > 0) key.v[12 + i - 1] = strides_bytes[i - 1];
  }
  {
    std::lock_guard<std::mutex> lk(g_tmap_mu);
    auto it = g_tmap_cache.find(key);
    if (it != g_tmap_cache.end()) {
      *out = it->second;
      return 0;
    }
  }
  // The encoder is a driver entry point and needs a current context; a thread that has made no runtime call yet (an autograd
  // worker whose first operation is a GEMM) has none. A runtime call binds the device's primary context to the thread; it is
  // made only when the thread has no context, because cudaFree is not allowed while a stream capture is in progress.
  {
    typedef CUresult (*CtxGetCurrentFn)(CUcontext*);
    static CtxGetCurrentFn get_ctx = nullptr;
    if (get_ctx == nullptr) {
      void* p = nullptr;
      cudaDriverEntryPointQueryResult q;
      if (cudaGetDriverEntryPoint("cuCtxGetCurrent", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
        get_ctx = reinterpret_cast<CtxGetCurrentFn>(p);
    }
    CUcontext ctx = nullptr;
    if (get_ctx == nullptr || get_ctx(&ctx) != CUDA_SUCCESS || ctx == nullptr) cudaFree(nullptr);
  }
  cuuint64_t gdim[5];
  cuuint64_t gstr[4];
  cuuint32_t bx[5], estr[5];
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bx[i] = box[i];
    estr[i] = 1;
    if (i > 0) {
      gstr[i - 1] = strides_bytes[i - 1];
      if (gstr[i - 1] % 16 != 0) return 903;
    }
  }
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)rank, const_cast<void*>(base), gdim, gstr, bx, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle_128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return 1000 + (int)r;
  {
    std::lock_guard<std::mutex> lk(g_tmap_mu);
    if (g_tmap_cache.size() >= kTmapCacheLimit) g_tmap_cache.clear();
    g_tmap_cache.emplace(key, *out);
  }
  return 0;
}

}  // namespace cb200
