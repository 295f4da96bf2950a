// GELU (tanh form) exactly as the reference evaluates it (cuda/gelu.cu:12-15): the literals are doubles, so the
// polynomial and the final product run in binary64 around a binary32 tanhf, and the result is narrowed to binary32
// before it is rounded to fp16.  Compiled by the same compiler with the same floating-point options, this is the
// reference's value for every fp16 input (pinned over all 65536 of them by tests/golden/reference_gelu_sm100.npz).
#pragma once

#include <cuda_fp16.h>

namespace cpmk {

__device__ __forceinline__ float gelu_reference(float x) {
    x = 0.5 * x * (1.0 + tanhf(0.7978845608028654 * x * (1.0 + 0.044715 * x * x)));
    return x;
}

__device__ __forceinline__ __half gelu_half(__half h) { return __float2half(gelu_reference(__half2float(h))); }

}  // namespace cpmk
