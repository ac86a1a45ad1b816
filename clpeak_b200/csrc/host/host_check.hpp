// Host references the backend checks its own readings against before reporting
// them ("computes real tiles on seeded operands and is checked against a host
// reference of the same math").  The reference project has nothing like this:
// its kernels run on constant operands and their outputs are never read back
// (src/cuda/compute_kernel.cpp:59-91).
//
// Plain C++, no fast-math: integer and checksum paths compare bit-exactly,
// floating tiles within the stated bound.
#pragma once

#include <cmath>
#include <cstdint>
#include <string>
#include <vector>

#include "../clpk_formats.h"
#include "../clpk_rng.h"
#include "../../../include/clpeak_b200_kernels.h"

namespace b200check {

inline float chainReference(float a, unsigned lane)
{
    float x = a;
    const float c = (float)lane;
    for (int i = 0; i < 128 * 16; ++i)
        x = std::fmaf(x, x, c);
    return x;
}

inline float seededChain(uint64_t seed, uint64_t item, float y, unsigned iters)
{
    float x[4];
    for (int l = 0; l < 4; ++l)
        x[l] = clpk_uniform_pm1(seed, 4 * item + (uint64_t)l);
    for (unsigned k = 0; k < iters; ++k)
        for (int l = 0; l < 4; ++l)
            x[l] = std::fmaf(x[l], y, x[l]);
    return ((x[0] + x[1]) + x[2]) + x[3];
}

inline bool sameFloat(float a, float b)
{
    if (std::isnan(a) && std::isnan(b))
        return true;
    return clpk_f32_bits(a) == clpk_f32_bits(b);
}

inline uint32_t xorWords(const void *p, size_t bytes)
{
    const uint32_t *w = static_cast<const uint32_t *>(p);
    uint32_t x = 0;
    for (size_t i = 0; i < bytes / 4; ++i)
        x ^= w[i];
    return x;
}

// Per-thread order of the reference read-and-sum kernel
// (src/cuda/cuda_kernels/global_bandwidth.cu:14-71) for one output element.
inline float readSumReference(const float *in, int width, uint64_t outIndex)
{
    const uint64_t block = outIndex / 256, lid = outIndex % 256;
    float lane[4] = {0, 0, 0, 0};
    uint64_t off = block * 256 * 16 + lid;
    for (int i = 0; i < 16; ++i, off += 256)
        for (int l = 0; l < width; ++l)
            lane[l] = lane[l] + in[off * width + l];
    float r = lane[0];
    for (int l = 1; l < width; ++l)
        r = r + lane[l];
    return r;
}

// ---- tensor tiles -------------------------------------------------------------------

inline int kindK(int kind)
{
    switch (kind) {
    case CLPK_MMA_F16: case CLPK_MMA_BF16: return 16;
    case CLPK_MMA_E4M3: case CLPK_MMA_E5M2: case CLPK_MMA_I8: return 32;
    default: return 64;
    }
}

inline double decodeOperand(int kind, const uint8_t *t, const uint8_t *sf, int row, int k)
{
    const int K = kindK(kind);
    switch (kind) {
    case CLPK_MMA_F16: return clpk_f16_decode(reinterpret_cast<const uint16_t *>(t)[row * K + k]);
    case CLPK_MMA_BF16: return clpk_bf16_decode(reinterpret_cast<const uint16_t *>(t)[row * K + k]);
    case CLPK_MMA_E4M3: return clpk_e4m3_decode(t[row * K + k]);
    case CLPK_MMA_E5M2: return clpk_e5m2_decode(t[row * K + k]);
    case CLPK_MMA_I8: return (double)reinterpret_cast<const int8_t *>(t)[row * K + k];
    default: {
        const uint8_t byte = t[(row * K + k) / 2];
        const float v = clpk_e2m1_decode((k & 1) ? (byte >> 4) : (byte & 0xF));
        const int blk = kind == CLPK_MMA_MXF4 ? 32 : 16;
        const uint8_t sb = sf[row * (K / blk) + k / blk];
        const float s = kind == CLPK_MMA_MXF4 ? clpk_ue8m0_decode(sb) : clpk_e4m3_decode(sb);
        return (double)v * (double)s;
    }
    }
}

// Compares one accumulator tile (128x256 32-bit words) after n instructions.
// int8: exact.  Floating kinds: |got - n*P| <= (n + K) * 2^-22 * n * S with
// P the exact product and S = sum|a||b| (truncating fp32 accumulation, at most
// two units in the last place lost per addition).  Returns an empty string when
// the tile passes, otherwise a description of the first failure.
inline std::string checkTile(int kind, const uint8_t *a, const uint8_t *b, const uint8_t *sfa, const uint8_t *sfb,
                             uint32_t n, const uint32_t *tile, double *worstRatio = nullptr)
{
    const int K = kindK(kind);
    std::vector<double> da(128 * (size_t)K), db(256 * (size_t)K);
    for (int r = 0; r < 128; ++r)
        for (int k = 0; k < K; ++k)
            da[r * K + k] = decodeOperand(kind, a, sfa, r, k);
    for (int r = 0; r < 256; ++r)
        for (int k = 0; k < K; ++k)
            db[r * K + k] = decodeOperand(kind, b, sfb, r, k);
    const double rel = ((double)n + K) * std::ldexp(1.0, -22);
    double worst = 0.0;
    for (int i = 0; i < 128; ++i)
        for (int j = 0; j < 256; ++j) {
            double p = 0.0, s = 0.0;
            for (int k = 0; k < K; ++k) {
                const double t = da[i * K + k] * db[j * K + k];
                p += t;
                s += std::fabs(t);
            }
            const uint32_t word = tile[i * 256 + j];
            if (kind == CLPK_MMA_I8) {
                const int32_t want = (int32_t)((uint32_t)(int32_t)p * n);
                if ((int32_t)word != want)
                    return "int32 accumulator differs at (" + std::to_string(i) + "," + std::to_string(j) + ")";
            } else {
                const double got = clpk_bits_f32(word);
                const double tol = rel * n * s + 1e-30;
                const double ratio = std::fabs(got - n * p) / tol;
                worst = std::max(worst, ratio);
                if (!(ratio <= 1.0))
                    return "accumulator off by " + std::to_string(ratio) + "x the bound at (" + std::to_string(i) +
                           "," + std::to_string(j) + ")";
            }
        }
    if (worstRatio)
        *worstRatio = worst;
    return {};
}

// One element of C = A B^T from quantised 16-bit / 8-bit operands, in double.
inline double gemmElement(int dtype, const void *a, const void *b, uint64_t k, uint64_t i, uint64_t j, double *absSum)
{
    double acc = 0.0, s = 0.0;
    for (uint64_t x = 0; x < k; ++x) {
        double va, vb;
        if (dtype == CLPK_DT_BF16) {
            va = clpk_bf16_decode(static_cast<const uint16_t *>(a)[i * k + x]);
            vb = clpk_bf16_decode(static_cast<const uint16_t *>(b)[j * k + x]);
        } else if (dtype == CLPK_DT_F16) {
            va = clpk_f16_decode(static_cast<const uint16_t *>(a)[i * k + x]);
            vb = clpk_f16_decode(static_cast<const uint16_t *>(b)[j * k + x]);
        } else {
            va = clpk_e4m3_decode(static_cast<const uint8_t *>(a)[i * k + x]);
            vb = clpk_e4m3_decode(static_cast<const uint8_t *>(b)[j * k + x]);
        }
        acc += va * vb;
        s += std::fabs(va * vb);
    }
    if (absSum)
        *absSum = s;
    return acc;
}

} // namespace b200check
