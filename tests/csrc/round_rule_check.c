/*
 * Exhaustive host-side proof of the division-free rounding rule in
 * cpm_kernels_b200/csrc/cpmk_round_rule.h: for every fp16 scale s in the rule's domain and every
 * finite fp16 x with |x| * r_up <= limit, "up == dn" implies that the low byte of dn equals the
 * reference expression (int8_t)nearbyintf((float)x / (float)s)  (cuda/gemm.cu:16), and "up != dn" implies that
 * up and dn are neighbouring integers of which the even one (cpmk_round_tie_even) equals that expression.
 *
 * Usage: round_rule_check <first_scale_bits> <last_scale_bits> <stride>
 * Prints "pairs=<n> ties=<t> mismatches=<k>" and exits 0 iff k == 0.
 */
#include <stdio.h>
#include <stdlib.h>
#include "cpmk_round_rule.h"

typedef _Float16 f16;
static float h2f(uint16_t b) { f16 h; memcpy(&h, &b, 2); return (float)h; }

int main(int argc, char **argv) {
    unsigned first = argc > 1 ? (unsigned)strtoul(argv[1], 0, 0) : 0x0400u;
    unsigned last = argc > 2 ? (unsigned)strtoul(argv[2], 0, 0) : 0x7bffu;
    unsigned stride = argc > 3 ? (unsigned)strtoul(argv[3], 0, 0) : 1u;
    unsigned long long pairs = 0, ties = 0, bad = 0;
    for (unsigned sb = first; sb <= last; sb += stride) {
        float s = h2f((uint16_t)sb);
        if (!cpmk_scale_in_domain(s)) continue;
        float r_up, r_dn;
        cpmk_round_prepare(s, &r_up, &r_dn);
        for (unsigned xb = 0; xb < 0x10000u; ++xb) {
            if ((xb & 0x7c00u) == 0x7c00u) continue;          /* inf / NaN are outside the domain */
            float x = h2f((uint16_t)xb);
            if (!cpmk_round_domain_ok(fabsf(x), r_up)) continue;
            ++pairs;
            uint32_t bits;
            int8_t want = (int8_t)nearbyintf(x / s);           /* |x/s| < 128: the cast is defined */
            if (cpmk_round_pair(x, r_up, r_dn, &bits)) {
                if ((int8_t)(uint8_t)(bits & 0xff) != want) {
                    if (bad < 10) fprintf(stderr, "mismatch x=%04x s=%04x got=%d want=%d\n", xb, sb, (int8_t)(bits & 0xff), want);
                    ++bad;
                }
            } else {
                /* disagreement inside the domain: an exact tie, resolved to the even neighbour */
                ++ties;
                float up = fmaf(x, r_up, CPMK_ROUND_MAGIC), dn = fmaf(x, r_dn, CPMK_ROUND_MAGIC);
                uint32_t got = cpmk_round_tie_even(cpmk_float_bits(up), cpmk_float_bits(dn));
                if (fabsf(up - dn) != 1.0f || (int8_t)(uint8_t)(got & 0xff) != want) {
                    if (bad < 10) fprintf(stderr, "tie mismatch x=%04x s=%04x up=%g dn=%g got=%d want=%d\n", xb, sb, up, dn, (int8_t)(got & 0xff), want);
                    ++bad;
                }
            }
        }
    }
    printf("pairs=%llu ties=%llu mismatches=%llu\n", pairs, ties, bad);
    return bad != 0;
}
