// Host-side construction of TMA tensor maps for 64 x 64 bf16 tiles with 128-byte swizzle.
// The driver entry point is resolved through the runtime so the library does not link
// against libcuda directly.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>

#include "gca_b200.h"

namespace gca {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = []() -> EncodeTiledFn {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess) return nullptr;
    if (q != cudaDriverEntryPointSuccess) return nullptr;
    return (EncodeTiledFn)f;
  }();
  return fn;
}

// Encoded tensor maps are kept in a small table keyed by everything that went into them
// (base pointer, extents, strides, box, swizzle): a training loop calls with the same few tensors
// over and over, and every launch used to re-encode 5 (forward) to 12 (backward) maps through the
// driver.  The table is shared by all threads of the process (one mutex; an entry is a plain
// 128-byte value that is copied out, so nothing is retained by pointer).
struct TileMapKey {
  const void* base;
  long long dims[5];
  long long strides[4];
  int box_d2;
  int swizzle;
  bool operator==(const TileMapKey& o) const {
    if (base != o.base || box_d2 != o.box_d2 || swizzle != o.swizzle) return false;
    for (int i = 0; i < 5; ++i) if (dims[i] != o.dims[i]) return false;
    for (int i = 0; i < 4; ++i) if (strides[i] != o.strides[i]) return false;
    return true;
  }
};
struct TileMapCache {
  static constexpr int SLOTS = 256;
  std::mutex mu;
  TileMapKey keys[SLOTS];
  CUtensorMap maps[SLOTS];
  bool used[SLOTS] = {};
  static unsigned slot_of(const TileMapKey& k) {
    unsigned long long h = reinterpret_cast<unsigned long long>(k.base) * 0x9E3779B97F4A7C15ull;
    for (int i = 0; i < 5; ++i) h = (h ^ (unsigned long long)k.dims[i]) * 0x100000001B3ull;
    for (int i = 0; i < 4; ++i) h = (h ^ (unsigned long long)k.strides[i]) * 0x100000001B3ull;
    h = (h ^ (unsigned long long)(k.box_d2 * 2 + k.swizzle)) * 0x100000001B3ull;
    return (unsigned)(h >> 40) % SLOTS;
  }
};
inline TileMapCache& tile_map_cache() {
  static TileMapCache c;
  return c;
}

// A bf16 tensor viewed as (d0 = 64 contiguous, d1, d2, d3, d4) with element strides s1..s4;
// every copy moves one (64 x 64 x 1 x 1 x 1) box, i.e. 64 rows of 128 bytes, swizzled.
// `box_d2` > 1 makes one copy fetch that many consecutive entries of axis d2 (e.g. the two
// heads of a pair: two 64 x 64 tiles land back to back in shared memory); entries past the
// end of the axis are filled with zeros.
inline int make_tile_map_5d(CUtensorMap* map, const void* base, int d0, int d1, int d2, int d3, int d4,
                            long long s1, long long s2, long long s3, long long s4, int box_d2 = 1,
                            bool swizzle128 = true) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return GCA_ERR_TMA;
  const long long dims_in[5] = {d0, d1, d2, d3, d4};
  long long str_in[4] = {s1, s2, s3, s4};
  TileMapKey key;
  key.base = base; key.box_d2 = box_d2; key.swizzle = swizzle128 ? 1 : 0;
  for (int i = 0; i < 5; ++i) key.dims[i] = dims_in[i];
  for (int i = 0; i < 4; ++i) key.strides[i] = str_in[i];
  TileMapCache& cache = tile_map_cache();
  const unsigned slot = TileMapCache::slot_of(key);
  {
    std::lock_guard<std::mutex> lock(cache.mu);
    if (cache.used[slot] && cache.keys[slot] == key) { *map = cache.maps[slot]; return 0; }
  }
  cuuint64_t dims[5];
  cuuint64_t strides[4];
  for (int i = 0; i < 5; ++i) dims[i] = (cuuint64_t)dims_in[i];
  for (int i = 0; i < 4; ++i) {
    // a dimension of extent 1 never advances: any legal stride will do
    if (dims_in[i + 1] == 1 && (str_in[i] <= 0 || (str_in[i] % 8) != 0)) str_in[i] = 64;
    if (str_in[i] <= 0 || (str_in[i] % 8) != 0) return GCA_ERR_STRIDE;
    strides[i] = (cuuint64_t)str_in[i] * 2;
  }
  const cuuint32_t box[5] = {64, 64, (cuuint32_t)box_d2, 1, 1};
  const cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return GCA_ERR_TMA;
  {
    std::lock_guard<std::mutex> lock(cache.mu);
    cache.keys[slot] = key; cache.maps[slot] = *map; cache.used[slot] = true;
  }
  return 0;
}

}  // namespace gca
