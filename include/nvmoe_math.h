/*
 * nvmoe_math.h — pinned scalar arithmetic shared by the CUDA kernels and the CPU checker.
 *
 * The reference router and SwiGLU shaders call GLSL exp/log/sqrt/tanh, whose precision a Vulkan
 * driver is free to choose.  To make route weights reproducible bit for bit between a CPU and a
 * GPU, every transcendental used on the routing path is written here once, out of operations that
 * IEEE-754 defines exactly (add, mul, fma, div, sqrt, integer bit moves), with every fused step
 * spelled as an explicit fma so that no compiler contraction can change the result.  The file is
 * plain C99 / CUDA C++ and is compiled by gcc (with -ffp-contract=off) and by nvcc.
 *
 * Bit helpers follow the reference shaders exactly:
 *   bf16 <-> f32           runtime-rs/shaders/moe_router_score_topk_batch1_bf16.comp.template:46-54
 *   E8M0 scale decode      runtime-rs/shaders/independent_sparse_moe_gate_up_batch1_mxfp4.comp.template:293-297
 *   E2M1 -> E4M3 table     same file :79-81,246-248 and nerve/quantized_transforms.py:34-51
 *   activation scale       same file :357-363 (rounded_fp8_scale)
 */
#ifndef NVMOE_MATH_H
#define NVMOE_MATH_H

#include <stdint.h>
#include <string.h>
#include <math.h>

#if defined(__CUDACC__)
#define NVMOE_HD __host__ __device__ __forceinline__
#else
#define NVMOE_HD static inline
#endif

#if defined(__CUDA_ARCH__)
#define NVMOE_FMUL(a, b) __fmul_rn((a), (b))
#define NVMOE_FADD(a, b) __fadd_rn((a), (b))
#define NVMOE_FSUB(a, b) __fsub_rn((a), (b))
#define NVMOE_FMA(a, b, c) __fmaf_rn((a), (b), (c))
#define NVMOE_FDIV(a, b) __fdiv_rn((a), (b))
#define NVMOE_FSQRT(a) __fsqrt_rn((a))
#else
#define NVMOE_FMUL(a, b) ((float)(a) * (float)(b))
#define NVMOE_FADD(a, b) ((float)(a) + (float)(b))
#define NVMOE_FSUB(a, b) ((float)(a) - (float)(b))
#define NVMOE_FMA(a, b, c) fmaf((a), (b), (c))
#define NVMOE_FDIV(a, b) ((float)(a) / (float)(b))
#define NVMOE_FSQRT(a) sqrtf((a))
#endif

NVMOE_HD uint32_t nvmoe_f32_bits(float v) {
#if defined(__CUDA_ARCH__)
    return __float_as_uint(v);
#else
    uint32_t b;
    memcpy(&b, &v, 4);
    return b;
#endif
}

NVMOE_HD float nvmoe_bits_f32(uint32_t b) {
#if defined(__CUDA_ARCH__)
    return __uint_as_float(b);
#else
    float v;
    memcpy(&v, &b, 4);
    return v;
#endif
}

/* bf16 helpers: round-to-nearest-even on the bit pattern, no NaN special case. */
NVMOE_HD float nvmoe_bf16_to_f32(uint32_t h) { return nvmoe_bits_f32((h & 0xffffu) << 16); }

NVMOE_HD uint32_t nvmoe_f32_to_bf16(float v) {
    uint32_t bits = nvmoe_f32_bits(v);
    uint32_t lsb = (bits >> 16) & 1u;
    return ((bits + 0x7fffu + lsb) >> 16) & 0xffffu;
}

NVMOE_HD float nvmoe_round_bf16(float v) { return nvmoe_bf16_to_f32(nvmoe_f32_to_bf16(v)); }

/* E8M0 power-of-two scale; byte 0 decodes to 2^-127 (a subnormal), 255 is not produced. */
NVMOE_HD float nvmoe_e8m0_to_f32(uint32_t b) {
    b &= 0xffu;
    return nvmoe_bits_f32(b == 0u ? 0x00400000u : (b << 23));
}

/* E2M1 nibble -> the E4M3 byte that holds the same value. */
NVMOE_HD uint32_t nvmoe_e2m1_to_e4m3_bits(uint32_t nibble) {
    const uint32_t table = 0x3c383000u;  /* 00 30 38 3c */
    const uint32_t table_hi = 0x4c484440u; /* 40 44 48 4c */
    uint32_t m = nibble & 7u;
    uint32_t mag = ((m < 4u ? table : table_hi) >> ((m & 3u) * 8u)) & 0xffu;
    return mag | ((nibble & 8u) << 4);
}

/* E2M1 nibble -> value (sign bit 3, magnitudes 0 .5 1 1.5 2 3 4 6). */
NVMOE_HD float nvmoe_e2m1_to_f32(uint32_t nibble) {
    uint32_t m = nibble & 7u;
    /* twice the magnitude is an integer: 0 1 2 3 4 6 8 12 */
    uint32_t twice = (m < 4u) ? m : ((m & 1u) ? (3u << ((m >> 1) - 1u)) : (1u << (m >> 1)));
    float v = 0.5f * (float)twice;
    return (nibble & 8u) ? -v : v;
}

/* E4M3 (fn variant: no infinity, S.1111.111 is NaN) byte -> f32. */
NVMOE_HD float nvmoe_e4m3_to_f32(uint32_t b) {
    uint32_t sign = (b & 0x80u) << 24;
    uint32_t e = (b >> 3) & 0xfu;
    uint32_t m = b & 7u;
    float mag;
    if (e == 0u) {
        mag = (float)m * 0.001953125f; /* m * 2^-9 */
    } else {
        mag = nvmoe_bits_f32(((e + 120u) << 23) | (m << 20));
    }
    return nvmoe_bits_f32(nvmoe_f32_bits(mag) | sign);
}

/* f32 -> E4M3 byte, round to nearest even, saturating to +-448. Input must not be NaN. */
NVMOE_HD uint32_t nvmoe_f32_to_e4m3(float v) {
    uint32_t bits = nvmoe_f32_bits(v);
    uint32_t sign = (bits >> 24) & 0x80u;
    uint32_t abs_bits = bits & 0x7fffffffu;
    float a = nvmoe_bits_f32(abs_bits);
    if (a >= 464.0f) return sign | 0x7eu; /* above the midpoint 448..480 rounds past max: saturate */
    if (a < 0.015625f) {
        /* subnormal range: multiples of 2^-9, RNE via the magic-number add */
        float shifted = NVMOE_FADD(a, 16384.0f); /* ulp of 16384 in f32 is 2^-9 */
        uint32_t q = nvmoe_f32_bits(shifted) & 0x7fffffu; /* integer count of 2^-9 */
        return sign | q;                                   /* q==8 encodes 2^-6, the first normal */
    }
    /* normal: keep 3 mantissa bits, RNE on the bit pattern */
    uint32_t lsb = (abs_bits >> 20) & 1u;
    uint32_t rounded = abs_bits + 0x7ffffu + lsb;
    uint32_t e = (rounded >> 23) - 120u; /* bias 127 -> bias 7 */
    uint32_t m = (rounded >> 20) & 7u;
    uint32_t out = (e << 3) | m;
    if (out > 0x7eu) out = 0x7eu;
    return sign | out;
}

/* Activation scale of the reference: the smallest power of two >= max(block_max, 1e-4) / 448. */
NVMOE_HD float nvmoe_rounded_fp8_scale(float block_max) {
    /* 2^ceil(log2(m / 448)) for m = max(block_max, 1e-4) without the division: 448 = 1.75 * 2^8, so with
     * m = f * 2^e (1 <= f < 2) the quotient is (f / 1.75) * 2^(e-8), which lies in (2^(e-9), 2^(e-8)] when
     * f <= 1.75 and in (2^(e-8), 2^(e-7)) when f > 1.75; the division rounds to nearest and cannot cross
     * either power of two. m >= 1e-4 is a normal number. */
    uint32_t bits = nvmoe_f32_bits(fmaxf(block_max, 1e-4f));
    uint32_t exponent = ((bits >> 23) & 0xffu) - 8u + ((bits & 0x7fffffu) > 0x600000u ? 1u : 0u);
    return nvmoe_bits_f32(exponent << 23);
}

/* The same scale as the E8M0 byte (exponent + 127) that a block-scaled MMA consumes. */
NVMOE_HD uint32_t nvmoe_rounded_fp8_scale_e8m0(float block_max) {
    return nvmoe_f32_bits(nvmoe_rounded_fp8_scale(block_max)) >> 23;
}

/* ---- pinned transcendentals -------------------------------------------------------------- */

/* 2^n * y for integer n in [-300, 300], done as two exact-or-once-rounded multiplies. */
NVMOE_HD float nvmoe_scalbn(float y, int n) {
    /* straight-line code (selects, no branches): a warp that evaluates many of these can overlap them */
    n = n > 254 ? 254 : n;
    n = n < -300 ? -300 : n;
    int n1 = n / 2;
    int n2 = n - n1;
    int low = (n2 + 127 > 0) ? 0 : 1; /* n2 in [-150,-127]: the second factor is built from two normal ones */
    float s1 = nvmoe_bits_f32((uint32_t)(n1 + 127) << 23);
    float s1_low = NVMOE_FMUL(s1, nvmoe_bits_f32((uint32_t)(n2 + 64 + 127) << 23));
    float s2 = nvmoe_bits_f32((uint32_t)(n2 + 127) << 23);
    s1 = low ? s1_low : s1;
    s2 = low ? nvmoe_bits_f32((uint32_t)(-64 + 127) << 23) : s2;
    return NVMOE_FMUL(NVMOE_FMUL(y, s1), s2);
}

/* exp(x): round-to-nearest range reduction by ln2 (two-part constant), degree-6 polynomial. */
NVMOE_HD float nvmoe_expf(float x) {
    /* Arguments outside the range (and NaN) run the same straight-line code on a clamped copy and are
     * replaced at the end; inside the range the clamp changes nothing. */
    float xc = fminf(fmaxf(x, -104.0f), 89.0f);
    float fn = floorf(NVMOE_FMA(xc, 1.44269504088896341f, 0.5f));
    float r = NVMOE_FMA(fn, -0.693359375f, xc);
    r = NVMOE_FMA(fn, 2.12194440e-4f, r);
    float p = 1.9875691500e-4f;
    p = NVMOE_FMA(p, r, 1.3981999507e-3f);
    p = NVMOE_FMA(p, r, 8.3334519073e-3f);
    p = NVMOE_FMA(p, r, 4.1665795894e-2f);
    p = NVMOE_FMA(p, r, 1.6666665459e-1f);
    p = NVMOE_FMA(p, r, 5.0000001201e-1f);
    float r2 = NVMOE_FMUL(r, r);
    float y = NVMOE_FADD(NVMOE_FMA(p, r2, r), 1.0f);
    y = nvmoe_scalbn(y, (int)fn);
    y = (x < -103.98f) ? 0.0f : y;
    y = (x > 88.72284f) ? nvmoe_bits_f32(0x7f800000u) : y;
    return (x != x) ? x : y;
}

/* log(x) for finite x > 0: mantissa in [sqrt(1/2), sqrt(2)), degree-8 polynomial. */
NVMOE_HD float nvmoe_logf(float x) {
    uint32_t bits = nvmoe_f32_bits(x);
    int e = 0;
    if ((bits >> 23) == 0u) { /* subnormal: scale up by 2^23 */
        x = NVMOE_FMUL(x, 8388608.0f);
        bits = nvmoe_f32_bits(x);
        e = -23;
    }
    e += (int)(bits >> 23) - 126;
    float m = nvmoe_bits_f32((bits & 0x007fffffu) | 0x3f000000u); /* [0.5, 1) */
    if (m < 0.707106781186547524f) {
        e -= 1;
        m = NVMOE_FSUB(NVMOE_FADD(m, m), 1.0f);
    } else {
        m = NVMOE_FSUB(m, 1.0f);
    }
    float z = NVMOE_FMUL(m, m);
    float p = 7.0376836292e-2f;
    p = NVMOE_FMA(p, m, -1.1514610310e-1f);
    p = NVMOE_FMA(p, m, 1.1676998740e-1f);
    p = NVMOE_FMA(p, m, -1.2420140846e-1f);
    p = NVMOE_FMA(p, m, 1.4249322787e-1f);
    p = NVMOE_FMA(p, m, -1.6668057665e-1f);
    p = NVMOE_FMA(p, m, 2.0000714765e-1f);
    p = NVMOE_FMA(p, m, -2.4999993993e-1f);
    p = NVMOE_FMA(p, m, 3.3333331174e-1f);
    float y = NVMOE_FMUL(NVMOE_FMUL(p, m), z);
    float fe = (float)e;
    y = NVMOE_FMA(fe, -2.12194440e-4f, y);
    y = NVMOE_FMA(z, -0.5f, y);
    float r = NVMOE_FADD(m, y);
    return NVMOE_FMA(fe, 0.693359375f, r);
}

/* tanh(x): odd polynomial below 0.625, (1-e)/(1+e) with e = exp(-2|x|) above. */
NVMOE_HD float nvmoe_tanhf(float x) {
    float a = fabsf(x);
    float r;
    if (a < 0.625f) {
        float z = NVMOE_FMUL(x, x);
        float p = -5.70498872745e-3f;
        p = NVMOE_FMA(p, z, 2.06390887954e-2f);
        p = NVMOE_FMA(p, z, -5.37397155531e-2f);
        p = NVMOE_FMA(p, z, 1.33314422036e-1f);
        p = NVMOE_FMA(p, z, -3.33332819422e-1f);
        return NVMOE_FMA(NVMOE_FMUL(p, z), x, x);
    }
    if (a > 9.1f) {
        r = 1.0f;
    } else {
        float e = nvmoe_expf(NVMOE_FMUL(-2.0f, a));
        r = NVMOE_FDIV(NVMOE_FSUB(1.0f, e), NVMOE_FADD(1.0f, e));
    }
    return x < 0.0f ? -r : r;
}

/* 1 / (1 + exp(-v)), the router and SwiGLU sigmoid of the reference shaders. */
NVMOE_HD float nvmoe_sigmoidf(float v) {
    return NVMOE_FDIV(1.0f, NVMOE_FADD(1.0f, nvmoe_expf(-v)));
}

/* max(v,0) + log(1 + exp(-|v|)) (moe_router_score_topk_batch1_bf16.comp.template:56-58). */
NVMOE_HD float nvmoe_softplusf(float v) {
    return NVMOE_FADD(fmaxf(v, 0.0f), nvmoe_logf(NVMOE_FADD(1.0f, nvmoe_expf(-fabsf(v)))));
}

/*
 * SwiGLU of the expert shaders (…gate_up_batch1_mxfp4.comp.template:773-787) with the two
 * extension knobs: alpha scales the sigmoid argument and up_offset is added to the up value.
 * alpha = 1, up_offset = 0 is the reference expression g / (1 + exp(-g)) * u.
 */
NVMOE_HD float nvmoe_swiglu(float gate_acc, float up_acc, float limit, float alpha, float up_offset) {
    float g = nvmoe_round_bf16(gate_acc);
    float u = nvmoe_round_bf16(up_acc);
    if (limit > 0.0f) {
        g = fminf(g, limit);
        u = fminf(fmaxf(u, -limit), limit);
    }
    float denom = NVMOE_FADD(1.0f, nvmoe_expf(-NVMOE_FMUL(alpha, g)));
    float act = NVMOE_FMUL(NVMOE_FDIV(g, denom), NVMOE_FADD(u, up_offset));
    return nvmoe_round_bf16(act);
}

#endif /* NVMOE_MATH_H */
