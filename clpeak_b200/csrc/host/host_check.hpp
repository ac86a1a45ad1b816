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
#include <cstring>
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

// ---- chains of the other element types (clpk_compute_chain) --------------------------------
// Bit pattern of what thread `tid` of any block stores: float bits for the half,
// half2, mixed and bf16 chains, double bits for the double chain, the int32 for the
// integer chains.

inline float throughHalf(float x) { return clpk_f16_decode(clpk_f16_encode(x)); }
inline float throughBf16(float x) { return clpk_bf16_decode(clpk_bf16_encode(x)); }
// One-rounding fp16 FMA: half x half is exact in double, so std::fma in double rounds the
// exact sum once, and 53 >= 2*11 + 2 bits keep the later rounding to half harmless.
inline float halfFma(float x, float c) { return throughHalf((float)std::fma((double)x, (double)x, (double)c)); }

inline int32_t dot4Bytes(uint32_t x, uint32_t y, int32_t acc)
{
    int64_t s = acc;
    for (int b = 0; b < 4; ++b)
        s += (int64_t)(int8_t)(x >> (8 * b)) * (int64_t)(int8_t)(y >> (8 * b));
    return (int32_t)(uint32_t)(uint64_t)s;
}

inline uint64_t typedChainBits(int chain, double a, unsigned tid)
{
    auto fbits = [](float v) { return (uint64_t)clpk_f32_bits(v); };
    switch (chain) {
    case CLPK_CHAIN_HALF: {
        float x0 = throughHalf((float)a), x1 = throughHalf((float)a + 1.0f);
        const float c = throughHalf((float)tid);
        for (int i = 0; i < 1024; ++i) {
            x0 = halfFma(x0, c);
            x1 = halfFma(x1, c);
        }
        return fbits(throughHalf(x0 + x1));
    }
    case CLPK_CHAIN_HALF2: {
        float x = throughHalf((float)a);
        const float c = throughHalf((float)tid);
        for (int i = 0; i < 1024; ++i)
            x = halfFma(x, c);
        return fbits(x + x);
    }
    case CLPK_CHAIN_DOUBLE: {
        double x = a;
        const double c = (double)tid;
        for (int i = 0; i < 2048; ++i)
            x = std::fma(x, x, c);
        uint64_t bits;
        std::memcpy(&bits, &x, sizeof bits);
        return bits;
    }
    case CLPK_CHAIN_MIXED:
    case CLPK_CHAIN_BF16: {
        const bool half = chain == CLPK_CHAIN_MIXED;
        auto through = [&](float v) { return half ? throughHalf(v) : throughBf16(v); };
        float x = through((float)a);
        const float c = through((float)tid);
        const int inner = half ? 16 : 128;
        for (int o = 0; o < 2048 / inner; ++o) {
            for (int i = 0; i < inner; ++i)
                x = std::fmaf(x, x, c);
            x = through(x);
        }
        return fbits(x);
    }
    case CLPK_CHAIN_INT32: {
        uint32_t x = (uint32_t)(int32_t)a;
        for (int i = 0; i < 2048; ++i)
            x = x * x + tid;
        return x;
    }
    default: {
        static const int offsets[4][8] = {{0}, {0, 7}, {0, 7, 13, 19}, {0, 11, 17, 23, 29, 31, 37, 41}};
        const int row = chain - CLPK_CHAIN_INT8_DOT1, chains = 1 << row, ai = (int)a;
        const uint32_t x = (uint32_t)(ai & 0xff) | ((uint32_t)((ai + 1) & 0xff) << 8) |
                           ((uint32_t)((ai + 2) & 0xff) << 16) | ((uint32_t)((ai + 3) & 0xff) << 24);
        uint32_t y[8], sum = 0;
        int32_t acc[8];
        for (int j = 0; j < chains; ++j) {
            y[j] = tid + (uint32_t)j;
            acc[j] = (int32_t)tid + offsets[row][j];
        }
        for (int o = 0; o < 64 / chains; ++o)
            for (int j = 0; j < chains; ++j)
                for (int i = 0; i < 16; ++i) {
                    acc[j] = dot4Bytes(x, y[j], acc[j]);
                    y[j] ^= (uint32_t)acc[j];
                }
        for (int j = 0; j < chains; ++j)
            sum += (uint32_t)acc[j];
        return sum;
    }
    }
}

// What thread gid of the shared-memory rotation ends with (64 rotations by one slot).
inline float localBandwidthReference(int width, uint64_t gid)
{
    const uint32_t g = (uint32_t)(gid / 256 * 256 + (gid % 256 + 64) % 256);
    float s = (float)g;
    for (int l = 1; l < width; ++l)
        s = s + (float)(g + (uint32_t)l);
    return s;
}

// What thread gid of the texture read stores: 16 texels at (gid + i*threads) % texels.
inline float imageBandwidthReference(uint64_t gid, uint64_t threads, uint64_t texels, uint64_t seed)
{
    float s[4] = {0, 0, 0, 0};
    for (int i = 0; i < 16; ++i) {
        const uint64_t px = (gid + (uint64_t)i * threads) % texels;
        for (int ch = 0; ch < 4; ++ch)
            s[ch] = s[ch] + clpk_uniform01(seed, 4 * px + (uint64_t)ch);
    }
    return ((s[0] + s[1]) + s[2]) + s[3];
}

// The tiled order: 8 x 32 texel tiles numbered along x; block b's fetch i reads tile (16 b + i) mod
// tiles; thread t of the block sits at (4 (w % 2) + l % 4, 8 (w / 2) + l / 4) in the tile, w = t / 32, l = t % 32.
inline float imageBandwidthTiledReference(uint64_t gid, uint32_t width, uint32_t height, uint64_t seed)
{
    const uint32_t tilesX = width / 8, nTiles = tilesX * (height / 32);
    const uint32_t block = (uint32_t)(gid / 256), inBlock = (uint32_t)(gid % 256), w = inBlock / 32, l = inBlock % 32;
    const uint32_t dx = (w % 2) * 4 + l % 4, dy = (w / 2) * 8 + l / 4;
    float s[4] = {0, 0, 0, 0};
    for (uint32_t i = 0; i < 16; ++i) {
        const uint32_t tile = (uint32_t)(((uint64_t)block * 16 + i) % nTiles);
        const uint64_t x = (uint64_t)(tile % tilesX) * 8 + dx, y = (uint64_t)(tile / tilesX) * 32 + dy;
        const uint64_t px = y * width + x;
        for (int ch = 0; ch < 4; ++ch)
            s[ch] = s[ch] + clpk_uniform01(seed, 4 * px + (uint64_t)ch);
    }
    return ((s[0] + s[1]) + s[2]) + s[3];
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
    case CLPK_MMA_TF32: return 8;
    case CLPK_MMA_F16: case CLPK_MMA_BF16: case CLPK_MMA_F16_F16: return 16;
    case CLPK_MMA_E4M3: case CLPK_MMA_E5M2: case CLPK_MMA_I8: case CLPK_MMA_E2M1: return 32;
    default: return 64;
    }
}

inline double decodeOperand(int kind, const uint8_t *t, const uint8_t *sf, int row, int k)
{
    const int K = kindK(kind);
    switch (kind) {
    case CLPK_MMA_F16: case CLPK_MMA_F16_F16:
        return clpk_f16_decode(reinterpret_cast<const uint16_t *>(t)[row * K + k]);
    case CLPK_MMA_TF32: return reinterpret_cast<const float *>(t)[row * K + k];
    case CLPK_MMA_E2M1: {
        const uint8_t byte = t[(row * K + k) / 2];
        return clpk_e2m1_decode((k & 1) ? (byte >> 4) : (byte & 0xF));
    }
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

// Compares one accumulator tile (128x256 32-bit words) after n instructions with
// the exact product of the decoded operands da[128][K], db[256][K].
// Integer kinds: exact.  Floating kinds: |got - n*P| <= (n + K) * 2^-22 * n * S with
// P the exact product and S = sum|a||b| (truncating fp32 accumulation, at most
// two units in the last place lost per addition).  Returns an empty string when
// the tile passes, otherwise a description of the first failure.
inline std::string checkDecodedTile(const std::vector<double> &da, const std::vector<double> &db, int K, bool integer,
                                    uint32_t n, const uint32_t *tile, double *worstRatio = nullptr)
{
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
            if (integer) {
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
    return checkDecodedTile(da, db, K, kind == CLPK_MMA_I8, n, tile, worstRatio);
}

// fp16-accumulate tile after ONE instruction: each output word holds a half in its low 16
// bits; it must lie within 2^-10 of the exact product relative to sum|a||b| (one rounding
// to half, plus whatever the data path loses before it).
inline std::string checkHalfAccumTile(const uint8_t *a, const uint8_t *b, const uint32_t *tile, double *worstRatio = nullptr)
{
    double worst = 0.0;
    for (int i = 0; i < 128; ++i)
        for (int j = 0; j < 256; ++j) {
            double p = 0.0, s = 0.0;
            for (int k = 0; k < 16; ++k) {
                const double t = (double)decodeOperand(CLPK_MMA_F16, a, nullptr, i, k) * (double)decodeOperand(CLPK_MMA_F16, b, nullptr, j, k);
                p += t;
                s += std::fabs(t);
            }
            const double got = clpk_f16_decode((uint16_t)(tile[i * 256 + j] & 0xFFFFu));
            const double ratio = std::fabs(got - p) / (std::ldexp(1.0, -10) * s + 1e-30);
            worst = std::max(worst, ratio);
            if (!(ratio <= 1.0))
                return "fp16 accumulator off by " + std::to_string(ratio) + "x the bound at (" + std::to_string(i) + "," +
                       std::to_string(j) + ")";
        }
    if (worstRatio)
        *worstRatio = worst;
    return {};
}

// ---- 2:4 sparse kinds ---------------------------------------------------------------------

// Keep the two largest magnitudes of every four along K (4-bit kinds: the two
// largest |x0|+|x1| of every four pairs); ties go to the lower index.  compressed
// is [rows][k/2] in K order, meta one nibble per group (first | second << 2), low
// nibble first.
// Expected sum of one warp's accumulator chains of the fp64 tensor probe (clpk_dmma_peak): chain j of warp w
// starts at w*CHAINS + j and adds A*B n times.  Exact for operands that are multiples of 2^-8 in [-1,1).
inline double dmmaExpected(const double *a, const double *b, uint32_t nMma, int warp, int row, int col)
{
    double p = 0;
    for (int k = 0; k < 4; ++k)
        p += a[row * 4 + k] * b[col * 4 + k];
    double init = 0;
    for (int j = 0; j < CLPK_DMMA_CHAINS; ++j)
        init += (double)(warp * CLPK_DMMA_CHAINS + j);
    return init + (double)CLPK_DMMA_CHAINS * (double)nMma * p;
}

inline void pruneTile(const std::vector<float> &dense, int rows, int k, bool pairs, std::vector<float> &compressed,
                      std::vector<uint8_t> &meta)
{
    const int unit = pairs ? 2 : 1, group = 4 * unit;
    compressed.assign((size_t)rows * k / 2, 0.0f);
    meta.assign((size_t)rows * k / (2 * group), 0);
    for (int r = 0; r < rows; ++r)
        for (int g = 0; g < k / group; ++g) {
            const float *x = &dense[(size_t)r * k + g * group];
            float mag[4];
            for (int u = 0; u < 4; ++u)
                mag[u] = pairs ? std::fabs(x[2 * u]) + std::fabs(x[2 * u + 1]) : std::fabs(x[u]);
            int first = 0;
            for (int u = 1; u < 4; ++u)
                if (mag[u] > mag[first]) first = u;
            int second = -1;
            for (int u = 0; u < 4; ++u)
                if (u != first && (second < 0 || mag[u] > mag[second])) second = u;
            const int s0 = std::min(first, second), s1 = std::max(first, second);
            float *c = &compressed[(size_t)r * k / 2 + g * 2 * unit];
            for (int e = 0; e < unit; ++e) {
                c[e] = x[s0 * unit + e];
                c[unit + e] = x[s1 * unit + e];
            }
            const uint8_t nib = (uint8_t)(s0 | (s1 << 2));
            uint8_t &mb = meta[(size_t)r * (k / (2 * group)) + g / 2];
            mb = (g & 1) ? (uint8_t)((mb & 0x0F) | (nib << 4)) : (uint8_t)((mb & 0xF0) | nib);
        }
}

inline int sparseK(int kind) { return (kind == CLPK_MMA_MXF4_SP || kind == CLPK_MMA_NVF4_SP) ? 128 : 64; }

inline std::string checkSparseTile(int kind, const uint8_t *aComp, const uint8_t *meta, const uint8_t *b,
                                   const uint8_t *sfa, const uint8_t *sfb, uint32_t n, const uint32_t *tile,
                                   double *worstRatio = nullptr)
{
    const int K = sparseK(kind);
    const bool fp4 = K == 128;
    const int nsf = kind == CLPK_MMA_NVF4_SP ? 4 : 2;
    auto scale = [&](const uint8_t *sf, int row, int kpos) -> double {
        const uint8_t sb = sf[row * nsf + kpos / (K / nsf)];
        return kind == CLPK_MMA_MXF4_SP ? clpk_ue8m0_decode(sb) : clpk_e4m3_decode(sb);
    };
    std::vector<double> da(128 * (size_t)K, 0.0), db(256 * (size_t)K);
    for (int r = 0; r < 128; ++r)
        for (int g = 0; g < 16; ++g) {
            const uint8_t byte = meta[r * 8 + g / 2];
            const int nib = (g & 1) ? (byte >> 4) : (byte & 0xF);
            const int sel[2] = {nib & 3, nib >> 2};
            if (!fp4) {
                for (int e = 0; e < 2; ++e) {
                    const int ci = r * 32 + 2 * g + e;
                    da[r * K + 4 * g + sel[e]] = kind == CLPK_MMA_I8_SP ? (double)reinterpret_cast<const int8_t *>(aComp)[ci]
                                                                       : (double)clpk_e4m3_decode(aComp[ci]);
                }
            } else {
                for (int e = 0; e < 4; ++e) {
                    const int ci = 4 * g + e;
                    const uint8_t cb = aComp[r * 32 + ci / 2];
                    const int kpos = 8 * g + 2 * sel[e / 2] + (e & 1);
                    da[r * K + kpos] = (double)clpk_e2m1_decode((ci & 1) ? (cb >> 4) : (cb & 0xF)) * scale(sfa, r, kpos);
                }
            }
        }
    for (int r = 0; r < 256; ++r)
        for (int k = 0; k < K; ++k) {
            if (!fp4)
                db[r * K + k] = kind == CLPK_MMA_I8_SP ? (double)reinterpret_cast<const int8_t *>(b)[r * K + k]
                                                      : (double)clpk_e4m3_decode(b[r * K + k]);
            else {
                const uint8_t bb = b[(r * K + k) / 2];
                db[r * K + k] = (double)clpk_e2m1_decode((k & 1) ? (bb >> 4) : (bb & 0xF)) * scale(sfb, r, k);
            }
        }
    return checkDecodedTile(da, db, K, kind == CLPK_MMA_I8_SP, n, tile, worstRatio);
}

// One element of C = A B^T from the quantised operands, in double.  NVFP4: packed
// e2m1 with row-major ue4m3 scales per 16 elements (sfa / sfb), tensor scales excluded.
inline double gemmElement(int dtype, const void *a, const void *b, uint64_t k, uint64_t i, uint64_t j, double *absSum,
                          const uint8_t *sfa = nullptr, const uint8_t *sfb = nullptr)
{
    double acc = 0.0, s = 0.0;
    for (uint64_t x = 0; x < k; ++x) {
        double va, vb;
        if (dtype == CLPK_DT_NVF4 || dtype == CLPK_DT_MXF4) {
            const bool mx = dtype == CLPK_DT_MXF4;
            const uint64_t blk = mx ? 32 : 16;
            const uint8_t ab = static_cast<const uint8_t *>(a)[(i * k + x) / 2], bb = static_cast<const uint8_t *>(b)[(j * k + x) / 2];
            const uint8_t sa = sfa[i * (k / blk) + x / blk], sb = sfb[j * (k / blk) + x / blk];
            va = (double)clpk_e2m1_decode((x & 1) ? (ab >> 4) : (ab & 0xF)) * (mx ? clpk_ue8m0_decode(sa) : clpk_e4m3_decode(sa));
            vb = (double)clpk_e2m1_decode((x & 1) ? (bb >> 4) : (bb & 0xF)) * (mx ? clpk_ue8m0_decode(sb) : clpk_e4m3_decode(sb));
        } else if (dtype == CLPK_DT_BF16) {
            va = clpk_bf16_decode(static_cast<const uint16_t *>(a)[i * k + x]);
            vb = clpk_bf16_decode(static_cast<const uint16_t *>(b)[j * k + x]);
        } else if (dtype == CLPK_DT_F16) {
            va = clpk_f16_decode(static_cast<const uint16_t *>(a)[i * k + x]);
            vb = clpk_f16_decode(static_cast<const uint16_t *>(b)[j * k + x]);
        } else if (dtype == CLPK_DT_I8) {
            va = static_cast<const int8_t *>(a)[i * k + x];
            vb = static_cast<const int8_t *>(b)[j * k + x];
        } else if (dtype == CLPK_DT_F32) {
            va = static_cast<const float *>(a)[i * k + x];
            vb = static_cast<const float *>(b)[j * k + x];
        } else if (dtype == CLPK_DT_F64) {
            va = static_cast<const double *>(a)[i * k + x];
            vb = static_cast<const double *>(b)[j * k + x];
        } else if (dtype == CLPK_DT_TF32) {
            va = clpk_bits_f32(static_cast<const uint32_t *>(a)[i * k + x] & 0xFFFFE000u);
            vb = clpk_bits_f32(static_cast<const uint32_t *>(b)[j * k + x] & 0xFFFFE000u);
        } else if (dtype == CLPK_DT_E5M2) {     // e5m2 A times e4m3 B
            va = clpk_e5m2_decode(static_cast<const uint8_t *>(a)[i * k + x]);
            vb = clpk_e4m3_decode(static_cast<const uint8_t *>(b)[j * k + x]);
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
