/* CPU oracle for the tiled scaled-dot-product-attention path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file restates, in plain C, the arithmetic of
 * the reference's CPU/CUDA kernels for the path so that the CUDA library can be
 * checked against it.  It is never linked into, loaded by or called from the
 * shipped library; only the test-suite, the smoke check and the CPU-baseline
 * leg of the benchmark use it.
 *
 * Parity pin: the fp32 functions are checked element-for-element against the
 * reference's own CPU kernels compiled from its sources (see build.py, target
 * `_ref`) and against the fp64 formulas of the reference's kernel tests; the
 * committed vectors under tests/golden/ were produced that way.
 *
 * Build: gcc -O2 -fPIC -shared -o libsdpa_oracle.so sdpa_oracle.c -lm
 * (no -ffast-math: the compensated sums rely on IEEE evaluation order).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* bfloat16 <-> float.  Round to nearest even; NaN stays NaN. */
static inline float bf16_to_f32(uint16_t h)
{
    uint32_t u = (uint32_t)h << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

static inline uint16_t f32_to_bf16(float f)
{
    uint32_t u;
    memcpy(&u, &f, 4);
    if((u & 0x7fffffffu) > 0x7f800000u)
    {
        return (uint16_t)((u >> 16) | 0x0040u);
    }
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

#define T float
#define LD(x) (x)
#define ST(x) (x)
#define FN(name) name##_f32
#include "ops_impl.inc"
#undef T
#undef LD
#undef ST
#undef FN

#define T uint16_t
#define LD(x) bf16_to_f32(x)
#define ST(x) f32_to_bf16(x)
#define FN(name) name##_bf16
#include "ops_impl.inc"
#undef T
#undef LD
#undef ST
#undef FN

/* IEEE half storage (the reference's fp16_t): conversions are the compiler's,
 * round to nearest even. */
#define T _Float16
#define LD(x) ((float)(x))
#define ST(x) ((_Float16)(x))
#define FN(name) name##_f16
#include "ops_impl.inc"
#undef T
#undef LD
#undef ST
#undef FN

/* Conversions exported for the Python side of the test-suite. */
void orc_f32_to_bf16(int64_t n, const float *src, uint16_t *dst)
{
    for(int64_t i = 0; i < n; ++i)
    {
        dst[i] = f32_to_bf16(src[i]);
    }
}

void orc_bf16_to_f32(int64_t n, const uint16_t *src, float *dst)
{
    for(int64_t i = 0; i < n; ++i)
    {
        dst[i] = bf16_to_f32(src[i]);
    }
}
