// Narrow floating-point codecs used by the set-up kernels and by the host-side
// result checks: e4m3 / e5m2 (OCP FP8), e2m1 (FP4), ue8m0 and ue4m3 scale
// factors, bf16 / fp16.  The reference project only hard-codes a few bit
// patterns of these formats (0x7F = 1.0 in ue8m0 and 0x38 = 1.0 in ue4m3 at
// src/cuda/cuda_blas.cpp:655-660; 0x3c bytes as fp8 / ue4m3 operands at
// src/cuda/cuda_kernels/wmma_nvf4_e2m1.cu:30-33); the definitions here follow
// the PTX ISA / OCP format tables.
#ifndef CLPK_FORMATS_H
#define CLPK_FORMATS_H

#include "clpk_rng.h"

// ---- e2m1: 1 sign, 2 exponent, 1 mantissa; magnitudes 0 .5 1 1.5 2 3 4 6 ------

CLPK_HD float clpk_e2m1_decode(uint8_t nib)
{
    const float mag[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};
    float m = mag[nib & 7];
    return (nib & 8) ? -m : m;
}

// Round to nearest, ties to the code with an even mantissa bit; saturates at 6.
CLPK_HD uint8_t clpk_e2m1_encode(float x)
{
    uint8_t sign = (clpk_f32_bits(x) >> 31) ? 8 : 0;
    float a = x < 0.0f ? -x : x;
    uint8_t code;
    if (!(a == a))           code = 7;   // NaN -> largest magnitude
    else if (a <= 0.25f)     code = 0;
    else if (a < 0.75f)      code = 1;
    else if (a <= 1.25f)     code = 2;
    else if (a < 1.75f)      code = 3;
    else if (a <= 2.5f)      code = 4;
    else if (a < 3.5f)       code = 5;
    else if (a <= 5.0f)      code = 6;
    else                     code = 7;
    return (uint8_t)(sign | code);
}

// ---- ue8m0: value = 2^(byte - 127) ------------------------------------------------

CLPK_HD float clpk_ue8m0_decode(uint8_t b)
{
    if (b == 0)
        return clpk_bits_f32(0x00400000u);      // 2^-127 (subnormal)
    return clpk_bits_f32((uint32_t)b << 23);
}

// Shared exponent for a block whose largest magnitude is amax:
// floor(log2(amax)) - 2, the 2 being the largest e2m1 exponent (OCP MX rule).
CLPK_HD uint8_t clpk_ue8m0_for_absmax(float amax)
{
    if (!(amax > 0.0f))
        return 127;
    int e = (int)(clpk_f32_bits(amax) >> 23) - 127;   // floor(log2) for normal floats
    if (e < -126)
        e = -126;
    int b = e - 2 + 127;
    if (b < 0)
        b = 0;
    if (b > 254)
        b = 254;
    return (uint8_t)b;
}

// ---- e4m3 (bias 7, no infinities, 0x7F/0xFF = NaN, max 448) ------------------------
// ue4m3 scale factors are e4m3 bytes with the sign bit clear.

CLPK_HD float clpk_e4m3_decode(uint8_t b)
{
    uint32_t s = b >> 7, e = (b >> 3) & 0xF, m = b & 7;
    float v;
    if (e == 0)
        v = (float)m * 0.001953125f;                                   // m * 2^-9
    else if (e == 15 && m == 7)
        v = clpk_bits_f32(0x7FC00000u);
    else
        v = clpk_bits_f32(((e + 120u) << 23) | (m << 20));            // 2^(e-7) * (1 + m/8)
    return s ? -v : v;
}

// ---- e5m2 (bias 15, IEEE-like: 0x7C = inf) --------------------------------------------

CLPK_HD float clpk_e5m2_decode(uint8_t b)
{
    uint32_t s = b >> 7, e = (b >> 2) & 0x1F, m = b & 3;
    float v;
    if (e == 0)
        v = (float)m * 1.52587890625e-05f;                             // m * 2^-16
    else if (e == 31)
        v = clpk_bits_f32(m ? 0x7FC00000u : 0x7F800000u);
    else
        v = clpk_bits_f32(((e + 112u) << 23) | (m << 21));
    return s ? -v : v;
}

// ---- bf16 / fp16 decode (host-side checks) ------------------------------------------------

CLPK_HD float clpk_bf16_decode(uint16_t h) { return clpk_bits_f32((uint32_t)h << 16); }

CLPK_HD float clpk_f16_decode(uint16_t h)
{
    uint32_t s = (uint32_t)(h >> 15) << 31, e = (h >> 10) & 0x1F, m = h & 0x3FF;
    if (e == 0) {
        float v = (float)m * 5.9604644775390625e-08f;                  // m * 2^-24
        return s ? -v : v;
    }
    if (e == 31)
        return clpk_bits_f32(s | 0x7F800000u | (m << 13));
    return clpk_bits_f32(s | ((e + 112u) << 23) | (m << 13));
}

// ---- bf16 / fp16 encode, round to nearest even (integer arithmetic only) ------------------

CLPK_HD uint16_t clpk_bf16_encode(float x)
{
    const uint32_t b = clpk_f32_bits(x);
    if ((b & 0x7FFFFFFFu) > 0x7F800000u)
        return (uint16_t)((b >> 16) | 0x40u);                          // quiet NaN
    return (uint16_t)((b + 0x7FFFu + ((b >> 16) & 1u)) >> 16);
}

CLPK_HD uint16_t clpk_f16_encode(float x)
{
    const uint32_t b = clpk_f32_bits(x), sign = (b >> 16) & 0x8000u, mag = b & 0x7FFFFFFFu;
    if (mag > 0x7F800000u)
        return (uint16_t)(sign | 0x7E00u);
    if (mag >= 0x477FF000u)                                            // rounds to >= 65520: infinity
        return (uint16_t)(sign | 0x7C00u);
    if (mag < 0x33000001u)                                             // <= 2^-25: rounds to zero
        return (uint16_t)sign;
    const int exp = (int)(mag >> 23) - 127;
    uint32_t man = (mag & 0x7FFFFFu) | 0x800000u;                      // 24-bit significand
    int shift = 13;                                                    // normal: keep 11 bits
    int he = exp + 15;
    if (he <= 0) {                                                     // subnormal half
        shift += 1 - he;
        he = 0;
    }
    const uint32_t kept = man >> shift, rem = man & ((1u << shift) - 1u), half = 1u << (shift - 1);
    uint32_t r = kept + ((rem > half || (rem == half && (kept & 1u))) ? 1u : 0u);
    // r carries the implicit bit for normals (bit 10); adding the exponent field handles the carry
    const uint32_t out = he > 0 ? (((uint32_t)(he - 1) << 10) + r) : r;
    return (uint16_t)(sign | out);
}

#endif // CLPK_FORMATS_H
