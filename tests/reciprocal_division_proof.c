/* Enumerates every pair (bf16 significand of x, F32 significand of d) and checks that
 *     r = RN(1 / d);  q = RN(x * r);  e = fma(-d, q, x);  q' = fma(e, r, q)
 * gives RN(x / d) bit for bit: the identity the pixel_norm / l2_normalize tile kernels use to divide a whole
 * column of bf16 values by one denominator without a division per element.  Signs are symmetric and a power of
 * two in x or d only shifts exponents (while everything stays normal), so the 2^7 x 2^23 pairs cover the domain
 * the kernels' range guards leave.  Prints "pairs N mismatches M"; exit status 1 if M != 0.
 * With argument "uncorrected" the last FMA is left out: the negative control (about a quarter must mismatch). */
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

static inline float as_float(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static inline uint32_t as_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }

int main(int argc, char** argv) {
    const int corrected = !(argc > 1 && strcmp(argv[1], "uncorrected") == 0);
    long mismatches = 0, pairs = 0;
#pragma omp parallel for reduction(+ : mismatches, pairs) schedule(dynamic, 1)
    for (uint32_t mx = 0; mx < 128; ++mx) {
        const float x = as_float(0x3f800000u | (mx << 16));
        for (uint32_t md = 0; md < (1u << 23); ++md) {
            const float d = as_float(0x3f800000u | md);
            const float r = 1.0f / d;
            const float q = x * r;
            const float e = fmaf(-d, q, x);
            const float fast = corrected ? fmaf(e, r, q) : q;
            pairs++;
            mismatches += as_bits(fast) != as_bits(x / d);
        }
    }
    printf("pairs %ld mismatches %ld\n", pairs, mismatches);
    return mismatches != 0;
}
