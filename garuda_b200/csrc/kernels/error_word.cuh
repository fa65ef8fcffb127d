// The device error word of one translation unit, and where the host learns of it.
//
// A kernel whose bounded wait runs out records a code here and winds down (it never traps and
// never spins for ever). The code goes to two places: a word in device memory, which
// `fetch_and_clear` reads with a synchronising copy, and, if the host has given one, a word in
// pinned host memory that the device can write to directly (`set_sink`). The engine reads that
// word where it already waits for a step's tokens, so that a failed step is noticed without another
// copy or synchronisation.
//
// Everything here is `static`: every .cu file that includes this header has a word and a sink of
// its own, and exports its own check.
#pragma once

#include <cuda_runtime.h>

namespace gb_err {

static __device__ int g_word;
static __device__ int* g_sink;       // pinned host memory, or null

__device__ __forceinline__ void report(int code) {
  atomicCAS(&g_word, 0, code);
  int* sink = g_sink;
  if (sink != nullptr) *reinterpret_cast<volatile int*>(sink) = code;
}

// The word's value (0: none), cleared if it was set; -1 if it cannot be read. Synchronises.
static inline int fetch_and_clear() {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_word, sizeof(int)) != cudaSuccess) return -1;
  if (v != 0) {
    int zero = 0;
    cudaMemcpyToSymbol(g_word, &zero, sizeof(int));
  }
  return v;
}

// `host_word`: pinned host memory (device-accessible under unified addressing), or null to stop.
static inline int set_sink(int* host_word) {
  return cudaMemcpyToSymbol(g_sink, &host_word, sizeof(host_word)) == cudaSuccess ? 0 : 1;
}

}  // namespace gb_err
