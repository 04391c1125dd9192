// Host-side helper: build (and cache) 2-D TMA tensor maps without linking libcuda.
// The driver entry point is fetched at run time, so the library also loads on a
// machine that has no GPU driver (the build host).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <atomic>
#include <mutex>
#include <unordered_map>

namespace blitz {

struct TmapKey {
  const void* ptr;
  uint64_t inner, outer, ld_bytes;
  uint32_t box_inner, box_outer, elem_bytes, swizzle;
  bool operator==(const TmapKey& o) const {
    return ptr == o.ptr && inner == o.inner && outer == o.outer && ld_bytes == o.ld_bytes &&
           box_inner == o.box_inner && box_outer == o.box_outer && elem_bytes == o.elem_bytes && swizzle == o.swizzle;
  }
};
struct TmapKeyHash {
  size_t operator()(const TmapKey& k) const {
    size_t h = reinterpret_cast<size_t>(k.ptr);
    auto mix = [&h](uint64_t v) { h ^= v + 0x9e3779b97f4a7c15ull + (h << 6) + (h >> 2); };
    mix(k.inner); mix(k.outer); mix(k.ld_bytes); mix(k.box_inner); mix(k.box_outer); mix(k.elem_bytes); mix(k.swizzle);
    return h;
  }
};

typedef CUresult (*PFN_encodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline PFN_encodeTiled get_encode_fn() {
  static PFN_encodeTiled fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_encodeTiled>(p);
  });
  return fn;
}

// Row-major 2-D tensor of 16-bit elements: `outer` rows of `inner` elements,
// row pitch `ld_bytes`.  Box = box_inner x box_outer elements.  swizzle_bytes
// is 128, 64, 32 or 0; box_inner * elem_bytes must equal swizzle_bytes when
// swizzling.  Out-of-range elements read as zero.  Returns false on failure.
inline bool get_tmap_2d(CUtensorMap* out, const void* ptr, uint64_t inner, uint64_t outer, uint64_t ld_bytes,
                        uint32_t box_inner, uint32_t box_outer, uint32_t elem_bytes = 2, uint32_t swizzle_bytes = 128) {
  static std::mutex mu;
  static std::unordered_map<TmapKey, CUtensorMap, TmapKeyHash> cache;
  TmapKey key{ptr, inner, outer, ld_bytes, box_inner, box_outer, elem_bytes, swizzle_bytes};
  {
    std::lock_guard<std::mutex> g(mu);
    auto it = cache.find(key);
    if (it != cache.end()) {
      *out = it->second;
      return true;
    }
  }
  PFN_encodeTiled enc = get_encode_fn();
  if (!enc) return false;
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) != 0 || (ld_bytes & 15) != 0) return false;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {ld_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMapSwizzle sw = swizzle_bytes == 128  ? CU_TENSOR_MAP_SWIZZLE_128B
                          : swizzle_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B
                          : swizzle_bytes == 32 ? CU_TENSOR_MAP_SWIZZLE_32B
                                                : CU_TENSOR_MAP_SWIZZLE_NONE;
  CUtensorMapDataType dt = elem_bytes == 2   ? CU_TENSOR_MAP_DATA_TYPE_UINT16
                           : elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_UINT32
                                             : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  CUtensorMap m;
  CUresult r = enc(&m, dt, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return false;
  {
    std::lock_guard<std::mutex> g(mu);
    if (cache.size() > 8192) cache.clear();
    cache.emplace(key, m);
  }
  *out = m;
  return true;
}

// 3-D tensor of 16-bit elements, dims (d0 fastest) with byte strides s1, s2 for
// d1, d2; box (b0, b1, b2); 128-byte swizzle (b0 * 2 bytes must be 128).
inline bool get_tmap_3d(CUtensorMap* out, const void* ptr, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t s1_bytes,
                        uint64_t s2_bytes, uint32_t b0, uint32_t b1, uint32_t b2) {
  static std::mutex mu;
  static std::unordered_map<TmapKey, CUtensorMap, TmapKeyHash> cache;
  TmapKey key{ptr, d0 * 1000003ull + d1, d2, s1_bytes * 1000003ull + s2_bytes, b0, b1 * 65536u + b2, 2, 128};
  {
    std::lock_guard<std::mutex> g(mu);
    auto it = cache.find(key);
    if (it != cache.end()) {
      *out = it->second;
      return true;
    }
  }
  PFN_encodeTiled enc = get_encode_fn();
  if (!enc) return false;
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) != 0 || (s1_bytes & 15) != 0 || (s2_bytes & 15) != 0) return false;
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {s1_bytes, s2_bytes};
  cuuint32_t box[3] = {b0, b1, b2};
  cuuint32_t estr[3] = {1, 1, 1};
  CUtensorMap m;
  CUresult r = enc(&m, CU_TENSOR_MAP_DATA_TYPE_UINT16, 3, const_cast<void*>(ptr), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return false;
  {
    std::lock_guard<std::mutex> g(mu);
    if (cache.size() > 8192) cache.clear();
    cache.emplace(key, m);
  }
  *out = m;
  return true;
}

// Number of SMs of the calling thread's current device (cached per device).
inline int device_sm_count() {
  static std::atomic<int> cache[64];
  int dev = 0;
  cudaGetDevice(&dev);
  const bool cacheable = dev >= 0 && dev < 64;
  int n = cacheable ? cache[dev].load(std::memory_order_relaxed) : 0;
  if (n == 0) {
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
    if (cacheable) cache[dev].store(n, std::memory_order_relaxed);
  }
  return n;
}

}  // namespace blitz
