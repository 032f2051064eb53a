// Entry point for callers that must not allocate device memory.
//
// This function has no counterpart in the reference project; it exists for
// hosts that embed this library but are not allowed to call cudaMalloc (or any
// allocating library routine) on the path where they need a gradient norm:
// for example a monitoring hook that runs between the micro-steps of a
// training job whose memory pool is fully reserved, a plug-in running inside
// a process whose allocator is owned by another framework, or code that runs
// after device memory has been deliberately filled.
#pragma once

#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Largest `n` accepted by tlm_sumsq_noalloc (elements).
#define TLM_SUMSQ_NOALLOC_MAX_N (1LL << 31)

// Return codes of tlm_sumsq_noalloc (0 = launched).
#define TLM_NOALLOC_ERR_TOO_LARGE (-101)   // n > TLM_SUMSQ_NOALLOC_MAX_N or n < 0
#define TLM_NOALLOC_ERR_SYMBOL (-102)      // cudaGetSymbolAddress / cudaGetDevice failed on this device
#define TLM_NOALLOC_ERR_ARGUMENT (-103)    // null pointer, or x not 16-byte aligned

// out[0] = sum_i x[i]^2 over n fp32 values on the device, like tlm_sumsq, but the
// per-block partial sums live in a fixed 4 KB array inside the library's device
// image instead of a caller-provided scratch buffer. Nothing is allocated or
// freed: no cudaMalloc, no cudaFree, no torch allocator.
//
//  * The array is part of every GPU context that loads the library and stays
//    there until the process exits.
//  * The first call on each device looks up the array's device address (with
//    that device current) and caches it; make that first call outside of any
//    stream capture. Later calls only launch two kernels on `stream`.
//  * All calls share the one array. Calls that may overlap on the GPU (different
//    streams without ordering) race on it; order them. Every launch overwrites
//    the entries it later reads, so nothing has to be cleared between calls.
//  * n above TLM_SUMSQ_NOALLOC_MAX_N is rejected with TLM_NOALLOC_ERR_TOO_LARGE
//    and nothing is launched. Positive return values are cudaError_t codes.
int tlm_sumsq_noalloc(const float* x, long long n, float* out, cudaStream_t stream);

// Human-readable text for a return code of tlm_sumsq_noalloc.
const char* tlm_noalloc_error_string(int code);

#ifdef __cplusplus
}
#endif
