// Host-side helpers of the tensor-core matrix products: tensor maps of row-major bfloat16 matrices
// (made once per matrix and box, then found again by address and shape) and the device's SM count.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <mutex>
#include <unordered_map>

#include "common.cuh"

namespace tc_host {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return (EncodeTiledFn)p;
  }();
  return fn;
}

struct MapKey {
  const void* ptr;
  long long rows, cols;
  int box_rows;
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && rows == o.rows && cols == o.cols && box_rows == o.box_rows;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    return std::hash<const void*>()(k.ptr) ^ (std::hash<long long>()(k.rows) * 31) ^
           (std::hash<long long>()(k.cols) * 131) ^ (size_t)k.box_rows * 7919;
  }
};

// A [rows, cols] bf16 row-major matrix seen through boxes of box_rows x 64, 128-byte swizzle.
inline int tensor_map_2d(const void* ptr, long long rows, long long cols, int box_rows, CUtensorMap* out) {
  static std::mutex mu;
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  MapKey key{ptr, rows, cols, box_rows};
  std::lock_guard<std::mutex> lock(mu);
  auto it = cache.find(key);
  if (it != cache.end()) {
    *out = it->second;
    return GB_OK;
  }
  EncodeTiledFn fn = encode_fn();
  if (!fn) return gb::fail(GB_CUDA_ERROR, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
  cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMap m;
  CUresult r = fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return gb::fail(GB_CUDA_ERROR, "cuTensorMapEncodeTiled failed with code %d for a %lld x %lld matrix", (int)r,
                    rows, cols);
  if (cache.size() > 4096) cache.clear();
  cache.emplace(key, m);
  *out = m;
  return GB_OK;
}

inline int sm_count() {
  static int n = [] {
    int dev = 0, v = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev);
    return v;
  }();
  return n;
}


}  // namespace tc_host
