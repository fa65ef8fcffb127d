// Shared by every kernel file: error reporting, dtype tags, conversions.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstring>

#define GB_EXPORT extern "C" __attribute__((visibility("default")))

// dtype tags of the C interface
enum GbDtype : int { GB_F32 = 0, GB_BF16 = 1 };

// Status codes returned by every entry point. 0 is success; the text of the
// last failure of the calling thread is available from gb_last_error().
enum GbStatus : int { GB_OK = 0, GB_BAD_ARGUMENT = 1, GB_CUDA_ERROR = 2, GB_UNSUPPORTED = 3 };

namespace gb {

inline char* error_buffer() {
  static thread_local char buf[512];
  return buf;
}

inline int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(error_buffer(), 512, fmt, ap);
  va_end(ap);
  return code;
}

inline int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(GB_CUDA_ERROR, "%s: %s", what, cudaGetErrorString(e));
  return GB_OK;
}

template <typename T>
__device__ __forceinline__ float to_float(T v);
template <>
__device__ __forceinline__ float to_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_float(float v);
template <>
__device__ __forceinline__ float from_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

}  // namespace gb

// One file of each library places this, so that the library exports the text
// of the calling thread's last failure.
#define GB_DEFINE_LAST_ERROR() \
  GB_EXPORT const char* gb_last_error() { return gb::error_buffer(); }

// Dispatch on a dtype tag: runs `body` with `T` bound to float or __nv_bfloat16.
#define GB_DISPATCH_DTYPE(tag, T, ...)                                   \
  [&]() -> int {                                                         \
    if ((tag) == GB_F32) { using T = float; return __VA_ARGS__(); }      \
    if ((tag) == GB_BF16) { using T = __nv_bfloat16; return __VA_ARGS__(); } \
    return gb::fail(GB_BAD_ARGUMENT, "unknown dtype tag %d", (int)(tag)); \
  }()
