// Device helpers shared by the quantisation kernels of the library (cpmk_quant.cu) and of the
// loadable kernel modules (modules/gemm_module.cu, modules/gemv_module.cu): scale from absmax, the rounding of
// eight fp16 values at a time, and the reference expression they fall back to.
#pragma once

#include <cuda_fp16.h>
#include <stdint.h>

#include "cpmk_round_rule.h"

namespace cpmk {

// half(amax / 127.0): the reference divides in double and narrows to float, then to half
// (cuda/gemm.cu:74).  A binary32 division gives the same float for every binary32 amax: x/127 has a
// period-7 binary expansion, so the double quotient never sits on a binary32 rounding boundary.
__device__ __forceinline__ __half scale_from_amax(float amax) { return __float2half_rn(__fdiv_rn(amax, 127.0f)); }

// The reference expression, used wherever the division-free rule does not apply.
__device__ __forceinline__ int8_t round_reference(float x, float s) { return (int8_t)nearbyintf(x / s); }

__device__ __forceinline__ float half2_max_to_float(__half2 m) { return __half2float(__hmax(__low2half(m), __high2half(m))); }

// max(|v|) over the 8 halves of a 128-bit vector, NaN elements dropped as fmaxf does.
__device__ __forceinline__ __half2 absmax8(const uint4 &v, __half2 m) {
    const __half2 *h = reinterpret_cast<const __half2 *>(&v);
    m = __hmax2(__habs2(h[0]), m);
    m = __hmax2(__habs2(h[1]), m);
    m = __hmax2(__habs2(h[2]), m);
    m = __hmax2(__habs2(h[3]), m);
    return m;
}

// The code of one element whose two roundings are `up_bits` and `dn_bits`: dn when they agree, else the even one of
// the two neighbouring integers (cpmk_round_tie_even).  Only for elements inside the rule's domain.
__device__ __forceinline__ uint32_t resolve_tie(uint32_t up_bits, uint32_t dn_bits) {
    return up_bits == dn_bits ? dn_bits : cpmk_round_tie_even(up_bits, dn_bits);
}

// Rounds the 8 halves of `v` with one scale.  r_up is NaN when the scale is outside the rule's
// domain, which sends every element to the reference expression.  The two roundings of each pair of
// elements are one packed fp32 FMA each (fma.rn.f32x2).
__device__ __forceinline__ uint2 round8_one_scale(const uint4 &v, float s, float r_up, float r_dn) {
    const __half2 *h = reinterpret_cast<const __half2 *>(&v);
    const float2 ru = make_float2(r_up, r_up), rd = make_float2(r_dn, r_dn);
    const float2 magic = make_float2(CPMK_ROUND_MAGIC, CPMK_ROUND_MAGIC);
    float2 dn[4];
    // disagreement between the two roundings is accumulated on the FMA pipe as a sum of squared differences
    // (zero iff every pair agrees; NaN -- from a NaN element or the out-of-domain marker -- propagates)
    float2 bad = make_float2(0.f, 0.f);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __half22float2(h[i]);
        const float2 up = __ffma2_rn(f, ru, magic);
        dn[i] = __ffma2_rn(f, rd, magic);
        const float2 d = __fadd2_rn(up, make_float2(-dn[i].x, -dn[i].y));
        bad = __ffma2_rn(d, d, bad);
    }
    uint32_t b[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        b[2 * i] = __float_as_uint(dn[i].x);
        b[2 * i + 1] = __float_as_uint(dn[i].y);
    }
    const float bad_sum = bad.x + bad.y;
    if (!(bad_sum == 0.f)) {
        if (bad_sum < 64.f) {
            // finite: the disagreements are exact ties (up = dn + 1), resolved to the even neighbour without a division
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 up = __ffma2_rn(__half22float2(h[i]), ru, magic);
                b[2 * i] = resolve_tie(__float_as_uint(up.x), b[2 * i]);
                b[2 * i + 1] = resolve_tie(__float_as_uint(up.y), b[2 * i + 1]);
            }
        } else {
            // NaN: a NaN / infinite element or a scale outside the rule's domain -- the reference expression itself
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 f = __half22float2(h[i]);
                b[2 * i] = (uint8_t)round_reference(f.x, s);
                b[2 * i + 1] = (uint8_t)round_reference(f.y, s);
            }
        }
    }
    uint2 out;
    out.x = __byte_perm(__byte_perm(b[0], b[1], 0x0040), __byte_perm(b[2], b[3], 0x0040), 0x5410);
    out.y = __byte_perm(__byte_perm(b[4], b[5], 0x0040), __byte_perm(b[6], b[7], 0x0040), 0x5410);
    return out;
}

}  // namespace cpmk
