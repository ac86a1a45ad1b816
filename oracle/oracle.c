/* CPU oracle for the clpeak_b200 kernels -- TEST INFRASTRUCTURE ONLY.
 * See oracle.h for scope and parity status ("parity unpinned" for kernel
 * values: the reference project holds no numeric golden vectors for this
 * path; its structural definitions are cited function by function).
 *
 * Compile with -ffp-contract=off -fno-fast-math: every float operation below
 * must be a single IEEE-754 rounding. */
#define _GNU_SOURCE
#include "oracle.h"

#include <math.h>
#include <pthread.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>

#pragma STDC FP_CONTRACT OFF

/* dtype / kind numbering mirrors include/clpeak_b200_kernels.h */
enum { DT_F32 = 0, DT_F16 = 1, DT_BF16 = 2, DT_E4M3 = 3, DT_E5M2 = 4, DT_I8 = 5, DT_MXF4 = 6, DT_NVF4 = 7,
       DT_MXF4_B64 = 8, DT_NVF4_B32 = 9, DT_TF32 = 10, DT_E2M1 = 11, DT_F64 = 12 };

static int fp4_block(int dtype) { return dtype == DT_MXF4 ? 32 : dtype == DT_NVF4 ? 16 : dtype == DT_MXF4_B64 ? 64 : 32; }
static int fp4_is_mx(int dtype) { return dtype == DT_MXF4 || dtype == DT_MXF4_B64; }
enum { MMA_F16 = 0, MMA_BF16 = 1, MMA_E4M3 = 2, MMA_E5M2 = 3, MMA_I8 = 4, MMA_MXF4 = 5, MMA_NVF4 = 6,
       MMA_E4M3_SP = 7, MMA_MXF4_SP = 8, MMA_NVF4_SP = 9, MMA_I8_SP = 10, MMA_TF32 = 11, MMA_F16_F16 = 12,
       MMA_E2M1 = 13 };

static uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

/* ------------------------------------------------------------------------- */
/* Generators.  splitmix64 twice: key = mix(seed), value = mix(key + idx).     */

static uint64_t mix64(uint64_t z)
{
    z += 0x9E3779B97F4A7C15ull;
    z ^= z >> 30; z *= 0xBF58476D1CE4E5B9ull;
    z ^= z >> 27; z *= 0x94D049BB133111EBull;
    z ^= z >> 31;
    return z;
}

uint64_t orc_rand64(uint64_t seed, uint64_t idx) { return mix64(mix64(seed) + idx); }

float orc_uniform01(uint64_t seed, uint64_t idx)
{
    return (float)(uint32_t)(orc_rand64(seed, idx) >> 40) * 0x1p-24f;
}

float orc_uniform_pm1(uint64_t seed, uint64_t idx)
{
    float t = (float)(uint32_t)(orc_rand64(seed, idx) >> 40) * 0x1p-23f;
    return t + -1.0f;
}

int orc_uniform_i4(uint64_t seed, uint64_t idx) { return (int)(orc_rand64(seed, idx) >> 60) - 8; }

/* ln(x) from IEEE operations only: x = m 2^e with m in [1/sqrt2, sqrt2),
 * ln m = 2 atanh t, t = (m-1)/(m+1), series to t^11. */
static float det_log(float x)
{
    uint32_t b = f2u(x);
    int e = (int)(b >> 23) - 127;
    float m = u2f((b & 0x007FFFFFu) | 0x3F800000u);
    if (m > 1.41421354f) { m = m * 0.5f; e += 1; }
    float t = (m + -1.0f) / (m + 1.0f);
    float s = t * t;
    float p = 0.0909090936f;
    p = fmaf(p, s, 0.111111112f);
    p = fmaf(p, s, 0.142857149f);
    p = fmaf(p, s, 0.2f);
    p = fmaf(p, s, 0.333333343f);
    p = fmaf(p, s, 1.0f);
    float lm = (2.0f * t) * p;
    return fmaf((float)e, 0.693147182f, lm);
}

/* cos(2 pi u), u in [0,1): fold to a quadrant, Taylor series in theta^2. */
static float det_cos2pi(float u)
{
    float q = u * 4.0f;
    int k = (int)q;
    float f = q + -(float)k;
    float th = f * 1.57079637f;
    float s = th * th;
    static const float cc[8] = {-1.14707454e-11f, 2.08767570e-09f, -2.75573192e-07f, 2.48015876e-05f,
                                -1.38888892e-03f, 4.16666679e-02f, -0.5f, 1.0f};
    static const float sc[8] = {-7.64716373e-13f, 1.60590438e-10f, -2.50521084e-08f, 2.75573188e-06f,
                                -1.98412701e-04f, 8.33333377e-03f, -0.166666672f, 1.0f};
    float c = cc[0], n = sc[0];
    for (int i = 1; i < 8; i++) { c = fmaf(c, s, cc[i]); n = fmaf(n, s, sc[i]); }
    n = n * th;
    switch (k & 3) {
    case 0: return c;
    case 1: return -n;
    case 2: return -c;
    default: return n;
    }
}

float orc_normal01(uint64_t seed, uint64_t idx)
{
    uint64_t h = orc_rand64(seed, idx);
    float u1 = (float)((uint32_t)(h >> 41) + 1u) * 0x1p-23f;     /* (0,1] */
    float u2 = (float)(uint32_t)(h & 0xFFFFFFu) * 0x1p-24f;      /* [0,1) */
    float r = sqrtf(-2.0f * det_log(u1));
    return r * det_cos2pi(u2);
}

void orc_fill_f32(float *dst, uint64_t first, uint64_t n, uint64_t seed, int dist, float mean, float std)
{
    for (uint64_t i = 0; i < n; i++) {
        uint64_t idx = first + i;
        if (dist == 0) dst[i] = orc_uniform01(seed, idx);
        else if (dist == 1) dst[i] = orc_uniform_pm1(seed, idx);
        else dst[i] = fmaf(std, orc_normal01(seed, idx), mean);
    }
}

void orc_fill_i8(int8_t *dst, uint64_t first, uint64_t n, uint64_t seed)
{
    for (uint64_t i = 0; i < n; i++) dst[i] = (int8_t)orc_uniform_i4(seed, first + i);
}

/* src/common/common.cpp:76-95 */
void orc_populate_reference(float *dst, uint64_t n)
{
    uint32_t st = 0xDEADBEEFu;
    for (uint64_t i = 0; i < n; i++) {
        st ^= st << 13; st ^= st >> 17; st ^= st << 5;
        dst[i] = u2f((st & 0x7F7FFFFFu) | 0x00800000u);
    }
}

/* ------------------------------------------------------------------------- */
/* Codecs                                                                     */

uint16_t orc_f32_to_bf16(float x)
{
    uint32_t b = f2u(x);
    if ((b & 0x7FFFFFFFu) > 0x7F800000u) return 0x7FFF;              /* NaN, as __float2bfloat16_rn */
    b += 0x7FFFu + ((b >> 16) & 1u);
    return (uint16_t)(b >> 16);
}

float orc_bf16_to_f32(uint16_t h) { return u2f((uint32_t)h << 16); }

/* Round |x| to a format with `mbits` mantissa bits and exponent bias `bias`
 * (ties to even); returns the magnitude code WITHOUT range handling: the
 * caller saturates.  Works in double, where every step is exact. */
static uint32_t small_encode_mag(double a, int ebits, int mbits, int bias)
{
    if (a == 0.0) return 0;
    int e;
    (void)frexp(a, &e);          /* a = f 2^e, f in [0.5,1) -> floor(log2 a) = e-1 */
    e -= 1;
    const int emin = 1 - bias;
    if (e < emin) e = emin;
    double q = ldexp(a, mbits - e);          /* in [2^mbits, 2^(mbits+1)) for normals */
    double r = nearbyint(q);                 /* default rounding mode: ties to even */
    uint32_t ri = (uint32_t)r;
    if (e == emin && ri < (1u << mbits))
        return ri;                           /* subnormal (exponent field 0) */
    if (ri == (2u << mbits)) { ri >>= 1; e += 1; }
    uint32_t efield = (uint32_t)(e + bias);
    (void)ebits;
    return (efield << mbits) | (ri & ((1u << mbits) - 1u));
}

uint8_t orc_f32_to_e4m3(float x)
{
    if (x != x) return 0x7F;
    uint8_t s = (f2u(x) >> 31) ? 0x80 : 0;
    double a = fabs((double)x);
    if (a > 448.0) return (uint8_t)(s | 0x7E);
    uint32_t m = small_encode_mag(a, 4, 3, 7);
    if (m > 0x7E) m = 0x7E;
    return (uint8_t)(s | m);
}

uint8_t orc_f32_to_e5m2(float x)
{
    if (x != x) return 0x7F;
    uint8_t s = (f2u(x) >> 31) ? 0x80 : 0;
    double a = fabs((double)x);
    if (a > 57344.0) return (uint8_t)(s | 0x7B);
    uint32_t m = small_encode_mag(a, 5, 2, 15);
    if (m > 0x7B) m = 0x7B;
    return (uint8_t)(s | m);
}

uint16_t orc_f32_to_f16(float x)
{
    uint32_t b = f2u(x);
    uint16_t s = (uint16_t)((b >> 16) & 0x8000u);
    if ((b & 0x7FFFFFFFu) > 0x7F800000u) return 0x7FFF;
    double a = fabs((double)x);
    if (isinf(a)) return (uint16_t)(s | 0x7C00);
    uint32_t m = small_encode_mag(a, 5, 10, 15);
    if (m >= 0x7C00) m = 0x7C00;             /* overflow -> infinity */
    return (uint16_t)(s | m);
}

float orc_f16_to_f32(uint16_t h)
{
    uint32_t e = (h >> 10) & 0x1F, m = h & 0x3FF;
    double v;
    if (e == 0) v = ldexp((double)m, -24);
    else if (e == 31) v = m ? NAN : INFINITY;
    else v = ldexp(1.0 + (double)m / 1024.0, (int)e - 15);
    return (float)((h & 0x8000) ? -v : v);
}

float orc_e4m3_to_f32(uint8_t b)
{
    uint32_t e = (b >> 3) & 0xF, m = b & 7;
    double v;
    if (e == 15 && m == 7) v = NAN;
    else if (e == 0) v = ldexp((double)m, -9);
    else v = ldexp(1.0 + (double)m / 8.0, (int)e - 7);
    return (float)((b & 0x80) ? -v : v);
}

float orc_e5m2_to_f32(uint8_t b)
{
    uint32_t e = (b >> 2) & 0x1F, m = b & 3;
    double v;
    if (e == 31) v = m ? NAN : INFINITY;
    else if (e == 0) v = ldexp((double)m, -16);
    else v = ldexp(1.0 + (double)m / 4.0, (int)e - 15);
    return (float)((b & 0x80) ? -v : v);
}

static const float kE2M1[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};

float orc_e2m1_to_f32(uint8_t nib)
{
    float v = kE2M1[nib & 7];
    return (nib & 8) ? -v : v;
}

uint8_t orc_f32_to_e2m1(float x)
{
    uint8_t s = (f2u(x) >> 31) ? 8 : 0;
    if (x != x) return (uint8_t)(s | 7);
    double a = fabs((double)x);
    /* nearest of the 8 magnitudes, ties to the even code */
    int best = 0;
    double bd = a;
    for (int c = 1; c < 8; c++) {
        double d = fabs(a - (double)kE2M1[c]);
        if (d < bd || (d == bd && (c & 1) == 0)) { bd = d; best = c; }
    }
    return (uint8_t)(s | best);
}

int8_t orc_f32_to_i8(float x)
{
    double r = nearbyint((double)x);
    if (r < -128.0) r = -128.0;
    if (r > 127.0) r = 127.0;
    return (int8_t)r;
}

float orc_ue8m0_to_f32(uint8_t b) { return (float)ldexp(1.0, (int)b - 127); }

uint8_t orc_ue8m0_for_absmax(float amax)
{
    if (!(amax > 0.0f)) return 127;
    int e;
    (void)frexpf(amax, &e);
    e -= 1;                                   /* floor(log2 amax) */
    if (e < -126) e = -126;                   /* subnormal inputs share the smallest normal exponent */
    int b = e - 2 + 127;
    if (b < 0) b = 0;
    if (b > 254) b = 254;
    return (uint8_t)b;
}

void orc_convert_f32(void *dst, const float *src, uint64_t n, int dtype)
{
    for (uint64_t i = 0; i < n; i++) {
        switch (dtype) {
        case DT_F16:  ((uint16_t *)dst)[i] = orc_f32_to_f16(src[i]); break;
        case DT_BF16: ((uint16_t *)dst)[i] = orc_f32_to_bf16(src[i]); break;
        case DT_E4M3: ((uint8_t *)dst)[i] = orc_f32_to_e4m3(src[i]); break;
        case DT_E5M2: ((uint8_t *)dst)[i] = orc_f32_to_e5m2(src[i]); break;
        case DT_I8:   ((int8_t *)dst)[i] = orc_f32_to_i8(src[i]); break;
        case DT_F64:  ((double *)dst)[i] = (double)src[i]; break;
        case DT_TF32: {     /* nearest even at bit 13; infinities and NaNs keep their class */
            uint32_t b; memcpy(&b, &src[i], 4);
            if ((b & 0x7F800000u) != 0x7F800000u) b += 0xFFFu + ((b >> 13) & 1u);
            ((uint32_t *)dst)[i] = b & 0xFFFFE000u;
            break;
        }
        case DT_E2M1: {     /* two per byte, even element in the low nibble (n even) */
            uint8_t nib = orc_f32_to_e2m1(src[i]);
            uint8_t *byte = &((uint8_t *)dst)[i / 2];
            *byte = (i & 1) ? (uint8_t)((*byte & 0x0F) | (nib << 4)) : nib;
            break;
        }
        default: break;
        }
    }
}

float orc_absmax_f32(const float *src, uint64_t n)
{
    float m = 0.0f;
    for (uint64_t i = 0; i < n; i++) { float a = fabsf(src[i]); if (a > m) m = a; }
    return m;
}

void orc_quantize_fp4(uint8_t *packed, uint8_t *scales, const float *src, uint64_t rows, uint64_t cols,
                      int dtype, float tensor_scale)
{
    const int blk = fp4_block(dtype);
    const uint64_t nblk = rows * cols / (uint64_t)blk;
    for (uint64_t b = 0; b < nblk; b++) {
        float v[64];
        float amax = 0.0f;
        for (int i = 0; i < blk; i++) {
            float x = src[b * blk + i];
            v[i] = fp4_is_mx(dtype) ? x : x / tensor_scale;
            float a = fabsf(v[i]);
            if (a > amax) amax = a;
        }
        uint8_t sb;
        float sd;
        if (fp4_is_mx(dtype)) { sb = orc_ue8m0_for_absmax(amax); sd = orc_ue8m0_to_f32(sb); }
        else { sb = orc_f32_to_e4m3(amax / 6.0f); sd = orc_e4m3_to_f32(sb); }
        scales[b] = sb;
        for (int i = 0; i < blk; i += 2) {
            uint8_t lo = 0, hi = 0;
            if (sd > 0.0f) { lo = orc_f32_to_e2m1(v[i] / sd); hi = orc_f32_to_e2m1(v[i + 1] / sd); }
            packed[b * (blk / 2) + i / 2] = (uint8_t)(lo | (hi << 4));
        }
    }
}

static double fp4_scale(const uint8_t *scales, uint64_t cols, int dtype, uint64_t row, uint64_t col)
{
    const int blk = fp4_block(dtype);
    uint8_t sb = scales[row * (cols / blk) + col / blk];
    return fp4_is_mx(dtype) ? (double)orc_ue8m0_to_f32(sb) : (double)orc_e4m3_to_f32(sb);
}

double orc_fp4_element(const uint8_t *packed, const uint8_t *scales, uint64_t cols, int dtype,
                       uint64_t row, uint64_t col)
{
    uint8_t byte = packed[(row * cols + col) / 2];
    uint8_t nib = (col & 1) ? (byte >> 4) : (byte & 0xF);
    return (double)orc_e2m1_to_f32(nib) * fp4_scale(scales, cols, dtype, row, col);
}

void orc_prune_2to4(float *compressed, uint8_t *meta, float *pruned, const float *dense, uint64_t rows, uint64_t k)
{
    for (uint64_t r = 0; r < rows; r++) {
        for (uint64_t g = 0; g < k / 4; g++) {
            const float *x = dense + r * k + g * 4;
            /* largest |x| first (lowest index on ties), then the largest of the rest */
            int first = 0;
            for (int i = 1; i < 4; i++) if (fabsf(x[i]) > fabsf(x[first])) first = i;
            int second = -1;
            for (int i = 0; i < 4; i++) {
                if (i == first) continue;
                if (second < 0 || fabsf(x[i]) > fabsf(x[second])) second = i;
            }
            int i0 = first < second ? first : second;
            int i1 = first < second ? second : first;
            compressed[r * (k / 2) + g * 2 + 0] = x[i0];
            compressed[r * (k / 2) + g * 2 + 1] = x[i1];
            uint8_t nib = (uint8_t)(i0 | (i1 << 2));
            uint8_t *mb = meta + r * (k / 8) + g / 2;
            if (g & 1) *mb = (uint8_t)((*mb & 0x0F) | (nib << 4));
            else *mb = (uint8_t)((*mb & 0xF0) | nib);
            if (pruned)
                for (int i = 0; i < 4; i++)
                    pruned[r * k + g * 4 + i] = (i == i0 || i == i1) ? x[i] : 0.0f;
        }
    }
}

/* ------------------------------------------------------------------------- */
/* Bandwidth                                                                   */

/* Thread (block, lid) reads 16 elements of `width` floats at element offsets
 * block*256*16 + lid + i*256, adds them lane-wise in that order starting from
 * zero, then sums the lanes left to right; out index = block*256 + lid. */
void orc_global_bandwidth(int width, const float *in, float *out, uint64_t n_floats)
{
    const uint64_t n_elems = n_floats / (uint64_t)width;
    const uint64_t blocks = n_elems / (256 * 16);
    for (uint64_t blk = 0; blk < blocks; blk++) {
        for (uint64_t lid = 0; lid < 256; lid++) {
            float sum[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            uint64_t off = blk * 256 * 16 + lid;
            for (int i = 0; i < 16; i++) {
                for (int l = 0; l < width; l++) sum[l] = sum[l] + in[off * width + l];
                off += 256;
            }
            float r = sum[0];
            for (int l = 1; l < width; l++) r = r + sum[l];
            out[blk * 256 + lid] = r;
        }
    }
}

uint32_t orc_xor_words(const void *src, uint64_t n_bytes)
{
    const uint32_t *w = (const uint32_t *)src;
    uint32_t x0 = 0, x1 = 0, x2 = 0, x3 = 0;
    uint64_t n = n_bytes / 4, i = 0;
    for (; i + 4 <= n; i += 4) { x0 ^= w[i]; x1 ^= w[i + 1]; x2 ^= w[i + 2]; x3 ^= w[i + 3]; }
    for (; i < n; i++) x0 ^= w[i];
    return x0 ^ x1 ^ x2 ^ x3;
}

void orc_triad(float *a, const float *b, const float *c, float s, uint64_t n)
{
    for (uint64_t i = 0; i < n; i++) {
        float t = s * c[i];
        a[i] = b[i] + t;
    }
}

typedef struct {
    int kind, tid, threads, passes;
    float *a; const float *b; const float *c; uint64_t n;
    pthread_barrier_t *bar;
    uint32_t x;
} stream_job_t;

static void *stream_worker(void *arg)
{
    stream_job_t *j = (stream_job_t *)arg;
    uint64_t per = (j->n / (uint64_t)j->threads) & ~(uint64_t)15;
    uint64_t lo = (uint64_t)j->tid * per;
    uint64_t hi = (j->tid == j->threads - 1) ? j->n : lo + per;
    pthread_barrier_wait(j->bar);
    for (int p = 0; p < j->passes; p++) {
        if (j->kind == 0) j->x ^= orc_xor_words(j->b + lo, (hi - lo) * 4);
        else if (j->kind == 1) memcpy(j->a + lo, j->b + lo, (hi - lo) * 4);
        else orc_triad(j->a + lo, j->b + lo, j->c + lo, 1.5f, hi - lo);
    }
    pthread_barrier_wait(j->bar);
    return NULL;
}

double orc_stream_pass_mt(int kind, float *a, const float *b, const float *c, uint64_t n, int threads,
                          int passes, uint32_t *xor_out)
{
    if (threads < 1) threads = 1;
    pthread_t *th = (pthread_t *)calloc((size_t)threads, sizeof(pthread_t));
    stream_job_t *jobs = (stream_job_t *)calloc((size_t)threads, sizeof(stream_job_t));
    pthread_barrier_t bar;
    pthread_barrier_init(&bar, NULL, (unsigned)threads + 1);
    for (int t = 0; t < threads; t++) {
        jobs[t] = (stream_job_t){kind, t, threads, passes, a, b, c, n, &bar, 0};
        pthread_create(&th[t], NULL, stream_worker, &jobs[t]);
    }
    struct timespec t0, t1;
    pthread_barrier_wait(&bar);
    clock_gettime(CLOCK_MONOTONIC, &t0);
    pthread_barrier_wait(&bar);
    clock_gettime(CLOCK_MONOTONIC, &t1);
    uint32_t x = 0;
    for (int t = 0; t < threads; t++) { pthread_join(th[t], NULL); x ^= jobs[t].x; }
    if (xor_out) *xor_out = x;
    pthread_barrier_destroy(&bar);
    free(th); free(jobs);
    double sec = (double)(t1.tv_sec - t0.tv_sec) + 1e-9 * (double)(t1.tv_nsec - t0.tv_nsec);
    return sec / (double)passes;
}

/* ------------------------------------------------------------------------- */
/* Chains                                                                      */

void orc_compute_sp(float *out, float a, uint64_t n_threads)
{
    for (uint64_t t = 0; t < n_threads; t++) {
        float x = a;
        float c = (float)(t % 256);
        for (int i = 0; i < 128 * 16; i++) x = fmaf(x, x, c);
        out[t] = x;
    }
}

/* The other shader-core chains, src/cuda/cuda_kernels/compute_hp.cu (scalar: two chains
 * x0 = A, x1 = A + 1; packed: both lanes A), compute_dp.cu, compute_mp.cu (value
 * through fp16 after every 16 FMAs), compute_bf16.cu (through bf16 after every 128),
 * compute_int32.cu (wrapping x*x + c) and compute_int8_dp.cu (a = dot4(x, y) + a;
 * y ^= a, chains taking turns in runs of 16).  chain = CLPK_CHAIN_*.  out: float
 * for chains 0, 1, 3, 4; double for 2; int32 for 5..9.  Thread t uses c = t % 256. */
static float half_round(float x) { return orc_f16_to_f32(orc_f32_to_f16(x)); }
static float bf16_round(float x) { return orc_bf16_to_f32(orc_f32_to_bf16(x)); }
/* fp16 FMA with one rounding: the product of two halves is exact in double, so the
 * double fma below is a correctly rounded sum of two doubles, and 53 >= 2*11 + 2 bits
 * make the second rounding (to half, through float: 24 >= 2*11 + 2) innocuous. */
static float half_fma(float x, float c) { return half_round((float)fma((double)x, (double)x, (double)c)); }

static int32_t dot4(uint32_t x, uint32_t y, int32_t a)
{
    int64_t s = a;
    for (int b = 0; b < 4; b++)
        s += (int64_t)(int8_t)(x >> (8 * b)) * (int64_t)(int8_t)(y >> (8 * b));
    return (int32_t)(uint32_t)(uint64_t)s;
}

void orc_compute_chain(int chain, void *out, double a, uint64_t n_threads)
{
    static const int dot_offsets[4][8] = {{0}, {0, 7}, {0, 7, 13, 19}, {0, 11, 17, 23, 29, 31, 37, 41}};
    for (uint64_t t = 0; t < n_threads; t++) {
        const uint32_t tid = (uint32_t)(t % 256);
        switch (chain) {
        case 0: {
            float x0 = half_round((float)a), x1 = half_round((float)a + 1.0f), c = half_round((float)tid);
            for (int i = 0; i < 1024; i++) { x0 = half_fma(x0, c); x1 = half_fma(x1, c); }
            ((float *)out)[t] = half_round(x0 + x1);      /* sum of two halves: exact in float, one rounding */
            break;
        }
        case 1: {
            float x = half_round((float)a), c = half_round((float)tid);
            for (int i = 0; i < 1024; i++) x = half_fma(x, c);
            ((float *)out)[t] = x + x;                    /* both lanes carry the same value */
            break;
        }
        case 2: {
            double x = a, c = (double)tid;
            for (int i = 0; i < 2048; i++) x = fma(x, x, c);
            ((double *)out)[t] = x;
            break;
        }
        case 3: {
            float x = half_round((float)a), c = half_round((float)tid);
            for (int o = 0; o < 128; o++) {
                for (int i = 0; i < 16; i++) x = fmaf(x, x, c);
                x = half_round(x);
            }
            ((float *)out)[t] = x;
            break;
        }
        case 4: {
            float x = bf16_round((float)a), c = bf16_round((float)tid);
            for (int o = 0; o < 16; o++) {
                for (int i = 0; i < 128; i++) x = fmaf(x, x, c);
                x = bf16_round(x);
            }
            ((float *)out)[t] = x;
            break;
        }
        case 5: {
            uint32_t x = (uint32_t)(int32_t)a;
            for (int i = 0; i < 2048; i++) x = x * x + tid;
            ((int32_t *)out)[t] = (int32_t)x;
            break;
        }
        default: {
            const int row = chain - 6, chains = 1 << row, ai = (int)a;
            const uint32_t x = (uint32_t)(ai & 0xff) | ((uint32_t)((ai + 1) & 0xff) << 8) |
                               ((uint32_t)((ai + 2) & 0xff) << 16) | ((uint32_t)((ai + 3) & 0xff) << 24);
            uint32_t y[8];
            int32_t acc[8];
            for (int j = 0; j < chains; j++) { y[j] = tid + (uint32_t)j; acc[j] = (int32_t)tid + dot_offsets[row][j]; }
            for (int o = 0; o < 64 / chains; o++)
                for (int j = 0; j < chains; j++)
                    for (int i = 0; i < 16; i++) { acc[j] = dot4(x, y[j], acc[j]); y[j] ^= (uint32_t)acc[j]; }
            uint32_t sum = 0;
            for (int j = 0; j < chains; j++) sum += (uint32_t)acc[j];
            ((int32_t *)out)[t] = (int32_t)sum;
            break;
        }
        }
    }
}

/* local_bandwidth_v1/v2/v4, src/cuda/cuda_kernels/local_bandwidth.cu: after 64 rotations
 * by one slot thread t holds the start value of thread (t + 64) % 256 of its block. */
void orc_local_bandwidth(int width, float *out, uint64_t n_threads)
{
    for (uint64_t t = 0; t < n_threads; t++) {
        const uint32_t g = (uint32_t)(t / 256 * 256 + (t % 256 + 64) % 256);
        float s = (float)g;
        for (int l = 1; l < width; l++) s = s + (float)(g + (uint32_t)l);
        out[t] = s;
    }
}

/* image_bandwidth, src/cuda/cuda_kernels/image_bandwidth.cu: 16 texel fetches per thread at
 * (gid + i * n_threads) % texels, channel-wise sums, then x + y + z + w.  Texel values are
 * the seeded uniform[0,1) stream, four per texel. */
void orc_image_bandwidth(float *out, uint64_t first, uint64_t count, uint64_t n_threads, uint64_t texels, uint64_t seed)
{
    for (uint64_t t = first; t < first + count; t++) {
        float s[4] = {0, 0, 0, 0};
        for (int i = 0; i < 16; i++) {
            const uint64_t px = (t + (uint64_t)i * n_threads) % texels;
            for (int ch = 0; ch < 4; ch++) s[ch] = s[ch] + orc_uniform01(seed, 4 * px + (uint64_t)ch);
        }
        out[t - first] = ((s[0] + s[1]) + s[2]) + s[3];
    }
}

/* The tiled order of the additive float4_tiled row: 8 x 32 texel tiles numbered along x; block b's
 * fetch i reads tile (16 b + i) mod tiles; thread t of a block sits at (4 (w % 2) + l % 4,
 * 8 (w / 2) + l / 4) inside the tile, w = t / 32, l = t % 32.  (No reference counterpart: its
 * kernel, src/cuda/cuda_kernels/image_bandwidth.cu:9-25, only has the strided order above.) */
void orc_image_bandwidth_tiled(float *out, uint64_t first, uint64_t count, uint32_t width, uint32_t height, uint64_t seed)
{
    const uint32_t tiles_x = width / 8, n_tiles = tiles_x * (height / 32);
    for (uint64_t t = first; t < first + count; t++) {
        const uint32_t block = (uint32_t)(t / 256), in_block = (uint32_t)(t % 256), w = in_block / 32, l = in_block % 32;
        const uint32_t dx = (w % 2) * 4 + l % 4, dy = (w / 2) * 8 + l / 4;
        float s[4] = {0, 0, 0, 0};
        for (uint32_t i = 0; i < 16; i++) {
            const uint32_t tile = (uint32_t)(((uint64_t)block * 16 + i) % n_tiles);
            const uint64_t x = (uint64_t)(tile % tiles_x) * 8 + dx, y = (uint64_t)(tile / tiles_x) * 32 + dy;
            const uint64_t px = y * width + x;
            for (int ch = 0; ch < 4; ch++) s[ch] = s[ch] + orc_uniform01(seed, 4 * px + (uint64_t)ch);
        }
        out[t - first] = ((s[0] + s[1]) + s[2]) + s[3];
    }
}

void orc_mad_chain(float *out, uint64_t first, uint64_t n_items, uint64_t seed, float y, uint32_t iters)
{
    for (uint64_t n = 0; n < n_items; n++) {
        uint64_t i = first + n;
        float x[4];
        for (int l = 0; l < 4; l++) x[l] = orc_uniform_pm1(seed, 4 * i + (uint64_t)l);
        for (uint32_t k = 0; k < iters; k++)
            for (int l = 0; l < 4; l++) x[l] = fmaf(x[l], y, x[l]);
        out[n] = ((x[0] + x[1]) + x[2]) + x[3];
    }
}

/* ------------------------------------------------------------------------- */
/* Pointer chase                                                               */

void orc_chase_cycle(uint32_t *next, uint64_t n, uint64_t seed)
{
    uint32_t *order = (uint32_t *)malloc(n * sizeof(uint32_t));
    for (uint64_t i = 0; i < n; i++) order[i] = (uint32_t)i;
    for (uint64_t i = n - 1; i > 0; i--) {               /* Sattolo: j strictly below i */
        uint64_t j = orc_rand64(seed, i) % i;
        uint32_t t = order[i]; order[i] = order[j]; order[j] = t;
    }
    for (uint64_t i = 0; i < n; i++) next[order[i]] = order[(i + 1) % n];
    free(order);
}

int orc_is_single_cycle(const uint32_t *next, uint64_t n)
{
    uint64_t steps = 0;
    uint32_t cur = 0;
    do {
        if (cur >= n) return 0;
        cur = next[cur];
        steps++;
    } while (cur != 0 && steps <= n);
    return steps == n;
}

void orc_chase(const uint32_t *next, uint32_t start, uint64_t hops, uint32_t *final_idx, uint32_t *xor_idx)
{
    uint32_t cur = start, x = 0;
    for (uint64_t h = 0; h < hops; h++) { cur = next[cur]; x ^= cur; }
    *final_idx = cur;
    *xor_idx = x;
}

/* ------------------------------------------------------------------------- */
/* Tensor tiles                                                                */

static int kind_k(int kind)
{
    switch (kind) {
    case MMA_TF32: return 8;
    case MMA_F16: case MMA_BF16: case MMA_F16_F16: return 16;
    case MMA_E4M3: case MMA_E5M2: case MMA_I8: case MMA_E2M1: return 32;
    default: return 64;
    }
}

static double decode_elem(int kind, const void *t, const uint8_t *sf, int row, int k, int K)
{
    switch (kind) {
    case MMA_F16: case MMA_F16_F16:
                   return (double)orc_f16_to_f32(((const uint16_t *)t)[row * K + k]);
    case MMA_TF32: return (double)((const float *)t)[row * K + k];
    case MMA_E2M1: {
        const uint8_t byte = ((const uint8_t *)t)[(row * K + k) / 2];
        return (double)orc_e2m1_to_f32((k & 1) ? (uint8_t)(byte >> 4) : (uint8_t)(byte & 0xF));
    }
    case MMA_BF16: return (double)orc_bf16_to_f32(((const uint16_t *)t)[row * K + k]);
    case MMA_E4M3: return (double)orc_e4m3_to_f32(((const uint8_t *)t)[row * K + k]);
    case MMA_E5M2: return (double)orc_e5m2_to_f32(((const uint8_t *)t)[row * K + k]);
    case MMA_I8:   return (double)((const int8_t *)t)[row * K + k];
    case MMA_MXF4: return orc_fp4_element((const uint8_t *)t, sf, (uint64_t)K, DT_MXF4, (uint64_t)row, (uint64_t)k);
    default:       return orc_fp4_element((const uint8_t *)t, sf, (uint64_t)K, DT_NVF4, (uint64_t)row, (uint64_t)k);
    }
}

void orc_mma_tile(int kind, const void *a, const void *b, const uint8_t *sfa, const uint8_t *sfb,
                  double *p_out, double *s_out)
{
    const int K = kind_k(kind);
    double *da = (double *)malloc(sizeof(double) * 128 * (size_t)K);
    double *db = (double *)malloc(sizeof(double) * 256 * (size_t)K);
    for (int r = 0; r < 128; r++) for (int k = 0; k < K; k++) da[r * K + k] = decode_elem(kind, a, sfa, r, k, K);
    for (int r = 0; r < 256; r++) for (int k = 0; k < K; k++) db[r * K + k] = decode_elem(kind, b, sfb, r, k, K);
    for (int i = 0; i < 128; i++)
        for (int j = 0; j < 256; j++) {
            double p = 0.0, s = 0.0;
            for (int k = 0; k < K; k++) { double t = da[i * K + k] * db[j * K + k]; p += t; s += fabs(t); }
            p_out[i * 256 + j] = p;
            if (s_out) s_out[i * 256 + j] = s;
        }
    free(da); free(db);
}

void orc_mma_tile_i8(const int8_t *a, const int8_t *b, uint32_t n_mma, int32_t *out)
{
    for (int i = 0; i < 128; i++)
        for (int j = 0; j < 256; j++) {
            int32_t p = 0;
            for (int k = 0; k < 32; k++) p += (int32_t)a[i * 32 + k] * (int32_t)b[j * 32 + k];
            out[i * 256 + j] = (int32_t)((uint32_t)p * n_mma);       /* two's-complement wrap */
        }
}


/* ------------------------------------------------------------------------- */
/* 2:4 sparse tiles                                                            */

/* 4-bit operands are pruned in pairs (one byte): of every four pairs along K the
 * two with the largest |x0|+|x1| are kept (ties: lower index).  compressed is
 * [rows][k/2] in K order, meta one nibble per group of eight logical positions
 * (pair index of the first kept pair | second << 2), two nibbles per byte. */
void orc_prune_pairs_2to4(float *compressed, uint8_t *meta, float *pruned, const float *dense, uint64_t rows, uint64_t k)
{
    for (uint64_t r = 0; r < rows; r++) {
        for (uint64_t g = 0; g < k / 8; g++) {
            const float *x = dense + r * k + g * 8;
            float mag[4];
            for (int p = 0; p < 4; p++) mag[p] = fabsf(x[2 * p]) + fabsf(x[2 * p + 1]);
            int first = 0;
            for (int p = 1; p < 4; p++) if (mag[p] > mag[first]) first = p;
            int second = -1;
            for (int p = 0; p < 4; p++) {
                if (p == first) continue;
                if (second < 0 || mag[p] > mag[second]) second = p;
            }
            int p0 = first < second ? first : second, p1 = first < second ? second : first;
            float *c = compressed + r * (k / 2) + g * 4;
            c[0] = x[2 * p0]; c[1] = x[2 * p0 + 1]; c[2] = x[2 * p1]; c[3] = x[2 * p1 + 1];
            uint8_t nib = (uint8_t)(p0 | (p1 << 2));
            uint8_t *mb = meta + r * (k / 16) + g / 2;
            if (g & 1) *mb = (uint8_t)((*mb & 0x0F) | (nib << 4));
            else *mb = (uint8_t)((*mb & 0xF0) | nib);
            if (pruned)
                for (int i = 0; i < 8; i++)
                    pruned[r * k + g * 8 + i] = (i / 2 == p0 || i / 2 == p1) ? x[i] : 0.0f;
        }
    }
}

static int sp_logical_k(int kind) { return (kind == MMA_MXF4_SP || kind == MMA_NVF4_SP) ? 128 : 64; }

/* Exact product tile of one sparse instruction: A is given compressed ([128][K/2]
 * elements in the kernel's encoding) with its selector nibbles; B is dense
 * [256][K].  Block-scaled kinds: sfa/sfb hold 2 (MXF4) or 4 (NVF4) factors per
 * row, factor j covering logical K positions [j*K/n, (j+1)*K/n). */
void orc_mma_tile_sp(int kind, const void *a_comp, const uint8_t *meta, const void *b, const uint8_t *sfa,
                     const uint8_t *sfb, double *p_out, double *s_out)
{
    const int K = sp_logical_k(kind);
    const int fp4 = (K == 128);
    const int nsf = kind == MMA_NVF4_SP ? 4 : 2;
    double *da = (double *)calloc((size_t)128 * K, sizeof(double));
    double *db = (double *)malloc(sizeof(double) * 256 * (size_t)K);
    for (int r = 0; r < 128; r++) {
        for (int g = 0; g < 16; g++) {
            const uint8_t byte = meta[r * 8 + g / 2];
            const int nib = (g & 1) ? (byte >> 4) : (byte & 0xF);
            const int s0 = nib & 3, s1 = nib >> 2;
            if (!fp4) {
                double v[2];
                for (int e = 0; e < 2; e++) {
                    const int ci = r * 32 + 2 * g + e;
                    v[e] = kind == MMA_I8_SP ? (double)((const int8_t *)a_comp)[ci]
                                             : (double)orc_e4m3_to_f32(((const uint8_t *)a_comp)[ci]);
                }
                da[r * K + 4 * g + s0] = v[0];
                da[r * K + 4 * g + s1] = v[1];
            } else {
                for (int e = 0; e < 4; e++) {
                    const int ci = 4 * g + e;                               /* compressed element index in the row */
                    const uint8_t cb = ((const uint8_t *)a_comp)[r * 32 + ci / 2];
                    const double val = orc_e2m1_to_f32((ci & 1) ? (cb >> 4) : (cb & 0xF));
                    const int pair = e < 2 ? s0 : s1;
                    const int kpos = 8 * g + 2 * pair + (e & 1);
                    const uint8_t sb = sfa[r * nsf + kpos / (K / nsf)];
                    const double sc = kind == MMA_MXF4_SP ? (double)orc_ue8m0_to_f32(sb) : (double)orc_e4m3_to_f32(sb);
                    da[r * K + kpos] = val * sc;
                }
            }
        }
    }
    for (int r = 0; r < 256; r++)
        for (int k = 0; k < K; k++) {
            if (!fp4) {
                db[r * K + k] = kind == MMA_I8_SP ? (double)((const int8_t *)b)[r * K + k]
                                                  : (double)orc_e4m3_to_f32(((const uint8_t *)b)[r * K + k]);
            } else {
                const uint8_t bb = ((const uint8_t *)b)[(r * K + k) / 2];
                const uint8_t sb = sfb[r * nsf + k / (K / nsf)];
                const double sc = kind == MMA_MXF4_SP ? (double)orc_ue8m0_to_f32(sb) : (double)orc_e4m3_to_f32(sb);
                db[r * K + k] = (double)orc_e2m1_to_f32((k & 1) ? (bb >> 4) : (bb & 0xF)) * sc;
            }
        }
    for (int i = 0; i < 128; i++)
        for (int j = 0; j < 256; j++) {
            double p = 0.0, s = 0.0;
            for (int k = 0; k < K; k++) { double t = da[i * K + k] * db[j * K + k]; p += t; s += fabs(t); }
            p_out[i * 256 + j] = p;
            if (s_out) s_out[i * 256 + j] = s;
        }
    free(da); free(db);
}

double orc_gemm_element(int dtype, const void *a, const void *b, const uint8_t *sfa, const uint8_t *sfb,
                        uint64_t k, uint64_t i, uint64_t j, double *abs_sum)
{
    double acc = 0.0, s = 0.0;
    for (uint64_t x = 0; x < k; x++) {
        double va, vb;
        switch (dtype) {
        case DT_BF16: va = orc_bf16_to_f32(((const uint16_t *)a)[i * k + x]); vb = orc_bf16_to_f32(((const uint16_t *)b)[j * k + x]); break;
        case DT_F16:  va = orc_f16_to_f32(((const uint16_t *)a)[i * k + x]);  vb = orc_f16_to_f32(((const uint16_t *)b)[j * k + x]); break;
        case DT_E4M3: va = orc_e4m3_to_f32(((const uint8_t *)a)[i * k + x]);  vb = orc_e4m3_to_f32(((const uint8_t *)b)[j * k + x]); break;
        /* the reference's "fp8_e5m2" GEMM row multiplies e5m2 A by e4m3 B (src/cuda/cuda_blas.cpp:632-638) */
        case DT_E5M2: va = orc_e5m2_to_f32(((const uint8_t *)a)[i * k + x]);  vb = orc_e4m3_to_f32(((const uint8_t *)b)[j * k + x]); break;
        case DT_I8:   va = ((const int8_t *)a)[i * k + x];                    vb = ((const int8_t *)b)[j * k + x]; break;
        /* the reference's "fp32" and "fp64" GEMM rows (src/cuda/cuda_blas.cpp:567-581): plain float / double operands */
        case DT_F32:  va = ((const float *)a)[i * k + x];                     vb = ((const float *)b)[j * k + x]; break;
        case DT_F64:  va = ((const double *)a)[i * k + x];                    vb = ((const double *)b)[j * k + x]; break;
        case DT_TF32: {   /* the multiplier reads sign, exponent and 10 mantissa bits of each fp32 word */
            uint32_t wa = ((const uint32_t *)a)[i * k + x] & 0xFFFFE000u, wb = ((const uint32_t *)b)[j * k + x] & 0xFFFFE000u;
            float fa, fb; memcpy(&fa, &wa, 4); memcpy(&fb, &wb, 4);
            va = fa; vb = fb;
            break;
        }
        default:
            va = orc_fp4_element((const uint8_t *)a, sfa, k, dtype, i, x);
            vb = orc_fp4_element((const uint8_t *)b, sfb, k, dtype, j, x);
            break;
        }
        acc += va * vb;
        s += fabs(va * vb);
    }
    if (abs_sum) *abs_sum = s;
    return acc;
}

/* src/common/common.cpp:35-45 */
unsigned orc_pick_iters(double per_iter_us, unsigned target_us, unsigned forced, unsigned max_iters)
{
    if (forced) return forced;
    if (target_us == 0) target_us = 5000000u;
    if (per_iter_us < 1.0) per_iter_us = 1.0;
    double want = (double)target_us / per_iter_us;
    if (want < 1.0) want = 1.0;
    if (want > (double)max_iters) want = (double)max_iters;
    return (unsigned)want;
}

/* fp64 tensor probe (clpk_dmma_peak): the successor of src/cuda/cuda_kernels/wmma_fp64.cu:15-46 (4 chains of
 * 1024 m8n8k4 instructions per warp on constant fragments) with seeded tiles.  Chain j of warp w starts at
 * w*chains + j in every element and runs n_mma instructions D = A*B + D; each instruction is replayed as
 * four fused multiply-adds in k order.  out[warps][8][8] = element-wise sum of a warp's chains.  For operands
 * that are multiples of 2^-8 in [-1,1) every step is exact, so the k order does not matter. */
void orc_dmma_tiles(const double *a, const double *b, uint32_t n_mma, int warps, int chains, double *out)
{
    for (int w = 0; w < warps; w++)
        for (int r = 0; r < 8; r++)
            for (int c = 0; c < 8; c++) {
                double sum = 0.0;
                for (int j = 0; j < chains; j++) {
                    double d = (double)(w * chains + j);
                    for (uint32_t i = 0; i < n_mma; i++)
                        for (int k = 0; k < 4; k++)
                            d = fma(a[r * 4 + k], b[c * 4 + k], d);
                    sum = j == 0 ? d : sum + d;
                }
                out[(w * 8 + r) * 8 + c] = sum;
            }
}
