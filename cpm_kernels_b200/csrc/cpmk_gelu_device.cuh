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

// The derivative, exactly as the reference evaluates it (cuda/gelu.cu:33-42): double literals again, so the cubic and
// the final sum run in binary64 around binary32 coshf / tanhf, sech2 is squared in binary32, and outside (-5, 5) the
// derivative is the step function.  grad = half(gelu'(x) * grad_out), one binary32 product.
__device__ __forceinline__ __half gelu_backward_half(__half grad_out, __half mat) {
    float v = __half2float(grad_out);
    float x = __half2float(mat);
    float gelu_grad;
    if (-5 < x && x < 5) {
        float x3 = x * x * x;
        float sech2 = 1.0 / coshf(0.797885 * x + 0.0356774 * x3);
        sech2 = sech2 * sech2;
        gelu_grad = 0.5 + (0.398942 * x + 0.0535161 * x3) * sech2 + 0.5 * tanhf(0.797885 * x + 0.0356774 * x3);
    } else {
        gelu_grad = x < 0 ? 0 : 1;
    }
    return __float2half(gelu_grad * v);
}

}  // namespace cpmk
