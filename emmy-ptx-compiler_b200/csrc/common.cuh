// Shared host-side plumbing of the kernel library: status codes, the per-thread error text,
// launch-error capture. Nothing here allocates device memory.
#pragma once
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/emmyb200.h"

namespace emmy {

// The message behind the last non-zero status returned to this host thread.
char* last_error_buffer();

inline int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(last_error_buffer(), 512, fmt, ap);
    va_end(ap);
    return code;
}

// A CUDA runtime error becomes a positive status (the cudaError_t value itself).
inline int cuda_fail(cudaError_t e, const char* what) {
    return fail((int)e, "%s: %s", what, cudaGetErrorString(e));
}

#define EMMY_CUDA(call)                                         \
    do {                                                        \
        cudaError_t e__ = (call);                               \
        if (e__ != cudaSuccess) return emmy::cuda_fail(e__, #call); \
    } while (0)

inline int launch_status(const char* kernel) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail((int)e, "launch of %s: %s", kernel, cudaGetErrorString(e));
    return EMMYB200_OK;
}

inline bool aligned(const void* p, size_t a) { return ((uintptr_t)p & (a - 1)) == 0; }

// Multiprocessor count of the current device (cached per device).
int sm_count();

}  // namespace emmy
