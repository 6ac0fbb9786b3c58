// Host-side helpers: TMA tensor-map encoding through the driver entry point (no libcuda link,
// so the library also loads on a machine without a driver), error plumbing, SM count.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include <mutex>
#include <unordered_map>

namespace lyra {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || !p) return nullptr;
    fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// rank-N tiled map over a row-major tensor. dims[0] is the innermost (contiguous) extent.
// strides_bytes[i] is the byte stride of dims[i+1]. Returns 0 on success.
inline int make_tmap(CUtensorMap* out, const void* base, CUtensorMapDataType dt, int rank, const uint64_t* dims,
                     const uint64_t* strides_bytes, const uint32_t* box, CUtensorMapSwizzle swz) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return -1;
  cuuint64_t d[5];
  cuuint64_t s[4];
  cuuint32_t b[5], e[5];
  for (int i = 0; i < rank; ++i) {
    d[i] = dims[i];
    b[i] = box[i];
    e[i] = 1;
  }
  for (int i = 0; i + 1 < rank; ++i) s[i] = strides_bytes[i];
  CUresult r = fn(out, dt, rank, const_cast<void*>(base), d, s, b, e, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    fprintf(stderr, "[lyra_b200] cuTensorMapEncodeTiled failed: %d (rank %d dims %llu,%llu box %u,%u stride %llu)\n", int(r), rank,
            (unsigned long long)dims[0], (unsigned long long)(rank > 1 ? dims[1] : 0), box[0], rank > 1 ? box[1] : 0,
            (unsigned long long)(rank > 1 ? strides_bytes[0] : 0));
    return -2;
  }
  return 0;
}

// The same, remembered: a training step encodes the same few hundred (address, shape, stride, box) combinations thousands of
// times (the caching allocator hands the activations of every microbatch the same blocks), and a map depends on nothing else,
// so a hit can never be stale. Encoding costs a driver call per operand of every GEMM launch; a hit costs a hash lookup.
struct TmapKey {
  const void* base;
  uint64_t dims[5], strides[4];
  uint32_t box[5];
  int dt, rank, swz;
  bool operator==(const TmapKey& o) const { return memcmp(this, &o, sizeof(TmapKey)) == 0; }
};
struct TmapKeyHash {
  size_t operator()(const TmapKey& k) const {
    const uint64_t* w = reinterpret_cast<const uint64_t*>(&k);
    uint64_t h = 1469598103934665603ull;
    for (size_t i = 0; i < sizeof(TmapKey) / 8; ++i) h = (h ^ w[i]) * 1099511628211ull;
    return static_cast<size_t>(h);
  }
};

inline int make_tmap_cached(CUtensorMap* out, const void* base, CUtensorMapDataType dt, int rank, const uint64_t* dims,
                            const uint64_t* strides_bytes, const uint32_t* box, CUtensorMapSwizzle swz) {
  static std::unordered_map<TmapKey, CUtensorMap, TmapKeyHash> cache;
  static std::mutex lock;
  TmapKey key;
  memset(&key, 0, sizeof(key));                  // padding bytes take part in the comparison
  key.base = base;
  key.dt = int(dt);
  key.rank = rank;
  key.swz = int(swz);
  for (int i = 0; i < rank; ++i) {
    key.dims[i] = dims[i];
    key.box[i] = box[i];
  }
  for (int i = 0; i + 1 < rank; ++i) key.strides[i] = strides_bytes[i];
  std::lock_guard<std::mutex> guard(lock);
  auto it = cache.find(key);
  if (it != cache.end()) {
    *out = it->second;
    return 0;
  }
  const int rc = make_tmap(out, base, dt, rank, dims, strides_bytes, box, swz);
  if (rc == 0) {
    if (cache.size() > (1u << 16)) cache.clear();
    cache.emplace(key, *out);
  }
  return rc;
}

inline int sm_count() {
  static int n = 0;
  if (!n) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

#define LYRA_CHECK_LAUNCH()                                                              \
  do {                                                                                   \
    cudaError_t e__ = cudaGetLastError();                                                \
    if (e__ != cudaSuccess) {                                                            \
      fprintf(stderr, "[lyra_b200] %s:%d launch failed: %s\n", __FILE__, __LINE__, cudaGetErrorString(e__)); \
      return -3;                                                                         \
    }                                                                                    \
  } while (0)

}  // namespace lyra
