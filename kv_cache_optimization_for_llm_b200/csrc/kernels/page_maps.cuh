// Tensor maps over a layer's pages of keys or values, for kernels that fetch whole pages by TMA.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <functional>
#include <mutex>
#include <unordered_map>

#include "common.cuh"

namespace kvb_page_maps {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
struct MapKey {
  const void* ptr; long long rows; int box, dh;
  bool operator==(const MapKey& o) const { return ptr == o.ptr && rows == o.rows && box == o.box && dh == o.dh; }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const { return std::hash<const void*>()(k.ptr) ^ (size_t)k.rows * 2654435761u ^ (size_t)k.box; }
};
inline std::mutex g_map_mutex;
inline std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_maps;

// The pages of one layer, [num_pages x nkv x page_size rows][head size] bfloat16, as a 2-D tensor
// map with boxes of box_rows x 64 and the 128-byte swizzle.  Rows beyond the last one read as zeros.
// Encoded once per address and shape.  ptr must be 16-byte aligned.
inline int pages_map(CUtensorMap* out, const void* ptr, long long rows, int box_rows, int dh) {
  static EncodeTiledFn fn = nullptr;
  std::lock_guard<std::mutex> lock(g_map_mutex);
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return KVB_ERR_BAD_SIZE;
    fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  MapKey key{ptr, rows, box_rows, dh};
  auto it = g_maps.find(key);
  if (it == g_maps.end()) {
    CUtensorMap m;
    cuuint64_t dims[2] = {(cuuint64_t)dh, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)dh * 2};
    cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return 1000 + (int)r;
    if (g_maps.size() > 4096) g_maps.clear();
    it = g_maps.emplace(key, m).first;
  }
  *out = it->second;
  return 0;
}

}  // namespace kvb_page_maps
