/*
 * Bit-reproducible scalar math shared by the CUDA router kernel and the CPU
 * checker.
 *
 * The router selects its top-k experts on softmax PROBABILITIES, so two
 * implementations agree on the selected ids only if every rounding on the way
 * from the logits to the probabilities is the same on both sides.  libm's expf
 * and the GPU's expf are each faithful but not identical, so the exponential is
 * written here once, out of IEEE-754 basic operations only (fused multiply-add,
 * add, multiply, all round-to-nearest-even, no flush-to-zero), which the host
 * compiler and the device execute identically.
 *
 * Reference behaviour being restated: `softmax_rows` subtracts the row maximum,
 * takes `exp`, sums left to right and multiplies by the reciprocal of the sum
 * (src/models/qwen3_6/forward.rs:793-806).  The reference calls its platform
 * libm for `exp`; this routine is a faithful (< 1 ulp) replacement.
 *
 * Build notes: host translation units that include this file must be compiled
 * without floating-point contraction or reassociation (-ffp-contract=off, no
 * -ffast-math).  On the device every operation is spelled with an explicit
 * rounding intrinsic, which the compiler never contracts.
 */
#ifndef FTM_EXACT_MATH_H
#define FTM_EXACT_MATH_H

#include <stdint.h>
#include <string.h>

#if defined(__CUDACC__)
#define FTM_HD __host__ __device__ __forceinline__
#else
#include <math.h>
#define FTM_HD static inline
#endif

#if defined(__CUDA_ARCH__)
#define FTM_FMA(a, b, c) __fmaf_rn((a), (b), (c))
#define FTM_ADD(a, b) __fadd_rn((a), (b))
#define FTM_MUL(a, b) __fmul_rn((a), (b))
#define FTM_RCP(a) __fdiv_rn(1.0f, (a))
#else
#define FTM_FMA(a, b, c) fmaf((a), (b), (c))
#define FTM_ADD(a, b) ((a) + (b))
#define FTM_MUL(a, b) ((a) * (b))
#define FTM_RCP(a) (1.0f / (a))
#endif

FTM_HD float ftm_bits_to_f32(uint32_t u) {
#if defined(__CUDA_ARCH__)
    return __uint_as_float(u);
#else
    float f;
    memcpy(&f, &u, 4);
    return f;
#endif
}

FTM_HD uint32_t ftm_f32_to_bits(float f) {
#if defined(__CUDA_ARCH__)
    return __float_as_uint(f);
#else
    uint32_t u;
    memcpy(&u, &f, 4);
    return u;
#endif
}

/* e^x for finite x; returns 0 below the subnormal range and +inf above the
 * float range.  Cody-Waite reduction x = n ln2 + r, |r| <= ln2/2, degree-7
 * polynomial in Horner form, then two exact power-of-two scalings so that
 * results in the subnormal range are rounded once. */
FTM_HD float ftm_expf(float x) {
    if (!(x > -104.0f)) return (x != x) ? x : 0.0f;
    if (x > 88.8f) return ftm_bits_to_f32(0x7f800000u);
    /* n = nearest integer to x / ln2, by the 1.5 * 2^23 shift trick */
    const float shift = 12582912.0f;
    float t = FTM_FMA(x, 1.44269504088896341f, shift);
    float n = FTM_ADD(t, -shift);
    float r = FTM_FMA(n, -0.693145751953125f, x);        /* ln2 high part: 0x3f317200 */
    r = FTM_FMA(n, -1.42860682030941723e-6f, r);         /* ln2 low part */
    /* Taylor coefficients 1/k!, k = 7..0; the truncation error r^8/8! is below
     * 6e-9 relative on |r| <= ln2/2, an order under half an ulp. */
    float p = 1.0f / 5040.0f;
    p = FTM_FMA(p, r, 1.0f / 720.0f);
    p = FTM_FMA(p, r, 1.0f / 120.0f);
    p = FTM_FMA(p, r, 1.0f / 24.0f);
    p = FTM_FMA(p, r, 1.0f / 6.0f);
    p = FTM_FMA(p, r, 0.5f);
    p = FTM_FMA(p, r, 1.0f);
    p = FTM_FMA(p, r, 1.0f);
    /* scale by 2^n in two exact steps: n = a + b with a = n/2 rounded */
    int ni = (int)n;
    int a = ni / 2;
    int b = ni - a;
    float sa = ftm_bits_to_f32((uint32_t)(a + 127) << 23);
    float sb = ftm_bits_to_f32((uint32_t)(b + 127) << 23);
    return FTM_MUL(FTM_MUL(p, sa), sb);
}

/* bf16 bit pattern -> f32 (src/domain/numerics.rs:6-8) */
FTM_HD float ftm_bf16_bits_to_f32(uint16_t b) { return ftm_bits_to_f32((uint32_t)b << 16); }

/* f32 -> bf16 bits, round to nearest even, NaN kept quiet.  This is the
 * narrowing the reference's adapter applies to host activations before launch
 * (src/infrastructure/cuda_moe.rs:63-66 uses half::bf16::from_f32). */
FTM_HD uint16_t ftm_f32_to_bf16_bits(float f) {
    uint32_t u = ftm_f32_to_bits(f);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u);
    uint32_t lsb = (u >> 16) & 1u;
    u += 0x7fffu + lsb;
    return (uint16_t)(u >> 16);
}

#endif /* FTM_EXACT_MATH_H */
