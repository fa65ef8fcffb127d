// Shared by every kernel file: error reporting, dtype tags, conversions.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
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

// A kernel attribute (the dynamic shared memory a kernel may use) belongs to a device: a flag that
// remembers "set" must be kept per device. `needed()` is true until `done()` has been called with
// the same device current. Not synchronised: two threads that make a kernel's first call on a
// device at the same moment both set the attribute, to the same value.
struct OncePerDevice {
  static constexpr int MAX_DEVICES = 64;
  bool set_[MAX_DEVICES] = {};
  static int device() {
    int d = 0;
    if (cudaGetDevice(&d) != cudaSuccess || d < 0 || d >= MAX_DEVICES) return -1;
    return d;
  }
  bool needed() const {
    const int d = device();
    return d < 0 || !set_[d];
  }
  void done() {
    const int d = device();
    if (d >= 0) set_[d] = true;
  }
};

// ---- programmatic dependent launch ----------------------------------------
// A kernel launched with launch_pdl may start while the kernel before it in the
// stream is still running. It must call pdl_wait() before it reads anything that
// kernel wrote and before it writes anything that kernel may still read; what it
// does before that (setting up barriers, fetching weights) overlaps the tail of
// its predecessor. pdl_launch_dependents() lets the kernel after it start early
// in the same way. Both are no-ops for a kernel launched the ordinary way.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

inline bool pdl_enabled() {
  static const bool on = [] {
    const char* v = getenv("GARUDA_B200_PDL");
    return !(v && v[0] == '0');
  }();
  return on;
}

// Launch with the programmatic-serialization attribute, and as clusters of the given shape if it
// holds more than one CTA.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              dim3 cluster, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attrs[2];
  int n = 0;
  if (pdl_enabled()) {
    attrs[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  if (cluster.x * cluster.y * cluster.z > 1) {
    attrs[n].id = cudaLaunchAttributeClusterDimension;
    attrs[n].val.clusterDim.x = cluster.x;
    attrs[n].val.clusterDim.y = cluster.y;
    attrs[n].val.clusterDim.z = cluster.z;
    ++n;
  }
  cfg.attrs = attrs;
  cfg.numAttrs = n;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

inline int check_pdl_launch(cudaError_t e, const char* what) {
  if (e != cudaSuccess) return fail(GB_CUDA_ERROR, "%s: %s", what, cudaGetErrorString(e));
  return check_launch(what);
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
