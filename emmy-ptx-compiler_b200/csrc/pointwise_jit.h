// Interface between the elementwise-program entry point and its compile-at-first-use form (pointwise_jit.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/emmyb200.h"

namespace emmy {

// Returned by pw_jit_launch when the program has to run on the interpreter instead: the specialised form is
// switched off, NVRTC cannot be loaded, or the program is an integer program.
constexpr int kPwJitUnavailable = 1 << 30;

// Launches the kernel specialised to `prog` (compiling it if this shape has not been seen), or returns
// kPwJitUnavailable. `group`: elements per thread and access group -- 8 or 4 when every non-broadcast buffer is
// aligned for accesses of that many elements, 0 for scalar accesses.
int pw_jit_launch(const emmyb200_pw_program& prog, const void* const* inputs, void* out, int64_t n, int group,
                  cudaStream_t stream);

}  // namespace emmy
