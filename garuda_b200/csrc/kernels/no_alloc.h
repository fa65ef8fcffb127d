// gb_sample_noalloc: sampling for callers that cannot allocate device memory.
//
// This entry point has no counterpart in hanumanit/garuda. It exists for hosts
// that embed the kernel library directly (through its C symbols, without the
// Python engine) and that must not call cudaMalloc while they run: a process
// that has already handed the whole device to its own memory pool, so that a
// further cudaMalloc would fail, or a latency-bound loop in which the implicit
// device-wide synchronisation of cudaMalloc and cudaFree would stall every
// other stream. gb_sample needs R * V floats of work space from its caller;
// gb_sample_noalloc brings its own, a fixed array that lives in the library's
// device image.
//
// Contract
//  * Same arguments and same result as gb_sample, without the scratch pointer:
//    one token per row of logits [R, V]; rows with temperature 0 are greedy.
//  * R * V must not exceed GB_SAMPLE_NOALLOC_MAX_FLOATS (2,097,152 floats,
//    8 MiB: 64 rows of a 32,000-entry vocabulary). Larger problems are refused
//    with GB_BAD_ARGUMENT and a message; nothing is launched.
//  * The work space is part of the library: every GPU on which the library is
//    loaded holds the 8 MiB until the process exits.
//  * The first call on a device looks up the array's device address
//    (cudaGetSymbolAddress, with that device current) and remembers it; later
//    calls on that device only launch. Make that first call before any stream
//    capture begins, and from one thread: the look-up is not synchronised.
//  * It calls neither cudaMalloc nor cudaFree nor any routine that allocates.
//  * All calls share the one array, and it keeps whatever the last call left.
//    Nothing in it has to start at zero: a call writes every element before it
//    reads it. Two calls that overlap on the GPU (different streams, no
//    ordering between them) race on the array and give wrong tokens; callers
//    order them.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#define GB_SAMPLE_NOALLOC_MAX_FLOATS (2 * 1024 * 1024)

#ifdef __cplusplus
extern "C" {
#endif

int gb_sample_noalloc(const float* logits, const float* temperature, const int32_t* top_k, const float* top_p,
                      const float* u, int32_t* out, int R, int V, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
