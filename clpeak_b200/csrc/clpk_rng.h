// Counter-based seeded generators shared by host and device code.
//
// clpeak itself fills buffers with a sequential xorshift32 stream
// (src/common/common.cpp:76-95 in the reference), which cannot be produced in
// parallel on a GPU nor replayed for one element.  Every value here is a pure
// function of (seed, element index), so a device kernel can fill 8 GiB in one
// pass and a host checker can regenerate any single element.
//
// Every floating-point step is one correctly-rounded IEEE-754 binary32
// operation (add, multiply, divide, square root, fused multiply-add) issued
// through the CLPK_F* macros, so host and device produce identical bits.
#ifndef CLPK_RNG_H
#define CLPK_RNG_H

#include <stdint.h>

#if defined(__CUDA_ARCH__)
#define CLPK_HD __host__ __device__ __forceinline__
#define CLPK_FMA(a, b, c) __fmaf_rn((a), (b), (c))
#define CLPK_FMUL(a, b) __fmul_rn((a), (b))
#define CLPK_FADD(a, b) __fadd_rn((a), (b))
#define CLPK_FDIV(a, b) __fdiv_rn((a), (b))
#define CLPK_FSQRT(a) __fsqrt_rn((a))
#else
#include <math.h>
#include <string.h>
#if defined(__CUDACC__)
#define CLPK_HD __host__ __device__ inline
#else
#define CLPK_HD static inline
#endif
#define CLPK_FMA(a, b, c) fmaf((a), (b), (c))
#define CLPK_FMUL(a, b) ((float)((float)(a) * (float)(b)))
#define CLPK_FADD(a, b) ((float)((float)(a) + (float)(b)))
#define CLPK_FDIV(a, b) ((float)((float)(a) / (float)(b)))
#define CLPK_FSQRT(a) sqrtf((a))
#endif

// splitmix64 finaliser.
CLPK_HD uint64_t clpk_mix64(uint64_t z)
{
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

// 64 random bits for element `idx` of stream `seed`.
CLPK_HD uint64_t clpk_rand64(uint64_t seed, uint64_t idx)
{
    return clpk_mix64(clpk_mix64(seed) + idx);
}

// uniform [0,1): 24 random bits, exactly representable.
CLPK_HD float clpk_uniform01(uint64_t seed, uint64_t idx)
{
    uint32_t k = (uint32_t)(clpk_rand64(seed, idx) >> 40);
    return CLPK_FMUL((float)k, 5.9604644775390625e-08f /* 2^-24 */);
}

// uniform [-1,1): k * 2^-23 - 1, exactly representable.
CLPK_HD float clpk_uniform_pm1(uint64_t seed, uint64_t idx)
{
    uint32_t k = (uint32_t)(clpk_rand64(seed, idx) >> 40);
    return CLPK_FADD(CLPK_FMUL((float)k, 1.1920928955078125e-07f /* 2^-23 */), -1.0f);
}

// uniform integer in [-8, 7].
CLPK_HD int clpk_uniform_i4(uint64_t seed, uint64_t idx)
{
    return (int)(clpk_rand64(seed, idx) >> 60) - 8;
}

CLPK_HD uint32_t clpk_f32_bits(float f)
{
#if defined(__CUDA_ARCH__)
    return __float_as_uint(f);
#else
    uint32_t u;
    memcpy(&u, &f, 4);
    return u;
#endif
}

CLPK_HD float clpk_bits_f32(uint32_t u)
{
#if defined(__CUDA_ARCH__)
    return __uint_as_float(u);
#else
    float f;
    memcpy(&f, &u, 4);
    return f;
#endif
}

// Natural log of a positive normal float from IEEE ops only:
// x = m * 2^e, m in [sqrt(1/2), sqrt(2)); ln m = 2 atanh((m-1)/(m+1)).
CLPK_HD float clpk_det_logf(float x)
{
    uint32_t b = clpk_f32_bits(x);
    int e = (int)(b >> 23) - 127;
    float m = clpk_bits_f32((b & 0x007FFFFFu) | 0x3F800000u);
    if (m > 1.41421354f) {
        m = CLPK_FMUL(m, 0.5f);
        e += 1;
    }
    float t = CLPK_FDIV(CLPK_FADD(m, -1.0f), CLPK_FADD(m, 1.0f));
    float s = CLPK_FMUL(t, t);
    float p = 0.0909090936f;            // 1/11
    p = CLPK_FMA(p, s, 0.111111112f);   // 1/9
    p = CLPK_FMA(p, s, 0.142857149f);   // 1/7
    p = CLPK_FMA(p, s, 0.2f);
    p = CLPK_FMA(p, s, 0.333333343f);
    p = CLPK_FMA(p, s, 1.0f);
    float lm = CLPK_FMUL(CLPK_FMUL(2.0f, t), p);
    return CLPK_FMA((float)e, 0.693147182f, lm);
}

// cos(2*pi*u) for u in [0,1) from IEEE ops only (quadrant fold + Taylor).
CLPK_HD float clpk_det_cos2pi(float u)
{
    float q = CLPK_FMUL(u, 4.0f);
    int k = (int)q;
    float f = CLPK_FADD(q, -(float)k);
    float th = CLPK_FMUL(f, 1.57079637f);
    float s = CLPK_FMUL(th, th);
    // cos(th)
    float c = -1.14707454e-11f;         // -1/14!
    c = CLPK_FMA(c, s, 2.08767570e-09f);
    c = CLPK_FMA(c, s, -2.75573192e-07f);
    c = CLPK_FMA(c, s, 2.48015876e-05f);
    c = CLPK_FMA(c, s, -1.38888892e-03f);
    c = CLPK_FMA(c, s, 4.16666679e-02f);
    c = CLPK_FMA(c, s, -0.5f);
    c = CLPK_FMA(c, s, 1.0f);
    // sin(th)
    float n = -7.64716373e-13f;         // -1/15!
    n = CLPK_FMA(n, s, 1.60590438e-10f);
    n = CLPK_FMA(n, s, -2.50521084e-08f);
    n = CLPK_FMA(n, s, 2.75573188e-06f);
    n = CLPK_FMA(n, s, -1.98412701e-04f);
    n = CLPK_FMA(n, s, 8.33333377e-03f);
    n = CLPK_FMA(n, s, -0.166666672f);
    n = CLPK_FMA(n, s, 1.0f);
    n = CLPK_FMUL(n, th);
    switch (k & 3) {
    case 0: return c;
    case 1: return -n;
    case 2: return -c;
    default: return n;
    }
}

// Standard normal deviate (Box-Muller, cosine branch) for element `idx`.
CLPK_HD float clpk_normal01(uint64_t seed, uint64_t idx)
{
    uint64_t h = clpk_rand64(seed, idx);
    uint32_t k1 = (uint32_t)(h >> 41);                // 23 bits
    uint32_t k2 = (uint32_t)(h & 0xFFFFFFu);          // 24 bits
    float u1 = CLPK_FMUL((float)(k1 + 1u), 1.1920928955078125e-07f);   // (0,1]
    float u2 = CLPK_FMUL((float)k2, 5.9604644775390625e-08f);          // [0,1)
    float r = CLPK_FSQRT(CLPK_FMUL(-2.0f, clpk_det_logf(u1)));
    return CLPK_FMUL(r, clpk_det_cos2pi(u2));
}

#endif // CLPK_RNG_H
