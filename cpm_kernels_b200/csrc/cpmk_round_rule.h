/*
 * The rounding rule of the quantisation kernels, shared between device code and the host-side
 * exhaustive check (tests/csrc/round_rule_check.c compiles this header with gcc).
 *
 * The reference rounds with an IEEE binary32 division per element (cuda/gemm.cu:16):
 *     q = (int8_t) nearbyintf((float)x / (float)s)           x, s fp16
 * A division costs ~10 issue slots; at 3 bytes of HBM traffic per element that is more than the
 * memory system leaves room for.  The rule below reproduces the same bits with two fused
 * multiply-adds and no division:
 *
 *     up = fma(x, r_up, M),  dn = fma(x, r_dn, M),   M = 1.5 * 2^23
 *     r_up = (1/s)(1 + 2^-20),  r_dn = (1/s)(1 - 2^-20)
 *
 * Adding M makes the fma itself round x*r to an integer (round-half-even, one rounding), and the
 * low byte of the result's bit pattern is that integer in two's complement.  Because x and s carry
 * 11-bit significands, a quotient x/s that is not exactly a half-integer lies at least 2^-12 away
 * from one, whereas the two perturbed products differ from x/s by at most ~2^-13: when up == dn
 * the common value is nearbyintf(x/s).  When they differ (exact ties, a handful per million) the
 * caller falls back to the reference expression itself.  tests/test_round_rule.py proves the claim
 * by enumeration over every (x, s) pair in the rule's domain.
 *
 * Domain (cpmk_round_domain_ok): s a normal finite fp16 (2^-14 <= s <= 65504), x finite,
 * |x| * r_up <= 127.75.  Outside it the caller uses the reference expression.
 */
#ifndef CPMK_ROUND_RULE_H_
#define CPMK_ROUND_RULE_H_

#include <stdint.h>

#if defined(__CUDACC__)
#define CPMK_RULE_FN __host__ __device__ __forceinline__
#else
#include <math.h>
#include <string.h>
#define CPMK_RULE_FN static inline
#endif

#define CPMK_ROUND_MAGIC 12582912.0f          /* 1.5 * 2^23, bit pattern 0x4B400000 */
#define CPMK_ROUND_UP    1.00000095367431640625f   /* 1 + 2^-20 */
#define CPMK_ROUND_DN    0.99999904632568359375f   /* 1 - 2^-20 */
#define CPMK_ROUND_LIMIT 127.75f

CPMK_RULE_FN uint32_t cpmk_float_bits(float v) {
#if defined(__CUDA_ARCH__)
    return __float_as_uint(v);
#else
    uint32_t b;
    memcpy(&b, &v, 4);
    return b;
#endif
}

/* s must be the fp16 scale widened to float. */
CPMK_RULE_FN int cpmk_scale_in_domain(float s) {
    return s >= 6.103515625e-05f && s <= 65504.0f;   /* false for NaN */
}

CPMK_RULE_FN void cpmk_round_prepare(float s, float *r_up, float *r_dn) {
    float r = 1.0f / s;                 /* IEEE division, once per row / column */
    *r_up = r * CPMK_ROUND_UP;
    *r_dn = r * CPMK_ROUND_DN;
}

/* amax = max |x| over the elements this scale will be applied to (finite, non-NaN). */
CPMK_RULE_FN int cpmk_round_domain_ok(float amax, float r_up) {
    return amax * r_up <= CPMK_ROUND_LIMIT;            /* false for NaN / inf */
}

/* Returns nonzero when the two roundings agree; *bits then holds the code in its low byte. */
CPMK_RULE_FN int cpmk_round_pair(float x, float r_up, float r_dn, uint32_t *bits) {
    float up = fmaf(x, r_up, CPMK_ROUND_MAGIC);
    float dn = fmaf(x, r_dn, CPMK_ROUND_MAGIC);
    *bits = cpmk_float_bits(dn);
    return up == dn;
}

/*
 * When the two roundings disagree inside the domain, x / s is an exact half-integer (anything else lies at least
 * 2^-12 away from one, further than the two perturbed products reach), up and dn are the two neighbouring integers,
 * and round-half-even picks the even one.  Adding the magic constant keeps the integer's parity in the lowest bit of
 * the bit pattern (1.5 * 2^23 is even), so the answer is dn when its lowest bit is clear and up otherwise.
 * Proven by the same enumeration as the rule itself (tests/csrc/round_rule_check.c).
 */
CPMK_RULE_FN uint32_t cpmk_round_tie_even(uint32_t up_bits, uint32_t dn_bits) {
    return (dn_bits & 1u) ? up_bits : dn_bits;
}

#endif /* CPMK_ROUND_RULE_H_ */
