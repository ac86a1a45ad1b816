// TEST DOUBLE for libclpeak_b200_kernels.so -- host-logic tests only.
//
// Implements the C ABI of include/clpeak_b200_kernels.h on the CPU, with
// CLPK_FAKE_DEVICES (default 1) pretend GPUs, so that the C++ host side (option
// parsing, the multi-device driver, the logger / FFI event stream, the result
// files) can be exercised by `pytest -m "not gpu"` on a machine without a GPU.
// It computes just enough for the backend's own result checks to pass on small
// sizes.  It is never linked into the product libraries.
#include <chrono>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <thread>
#include <vector>

#include "../../include/clpeak_b200_kernels.h"
#include "../../clpeak_b200/csrc/clpk_formats.h"
#include "../../clpeak_b200/csrc/clpk_rng.h"
// the new chain / shared-memory / texture rows reuse the backend's own host references: this double
// exercises the host plumbing, the numerics are pinned on the GPU against the oracle
#include "../../clpeak_b200/csrc/host/host_check.hpp"

namespace {
thread_local char g_err[256] = "";
thread_local int g_dev = 0;

int fakeDevices()
{
    const char *e = std::getenv("CLPK_FAKE_DEVICES");
    return e ? std::atoi(e) : 1;
}

int fail(int code, const char *msg)
{
    std::snprintf(g_err, sizeof(g_err), "%s", msg);
    return code;
}

// Generic round-to-nearest-even encoder for small formats (magnitude code only).
uint32_t encodeMag(double a, int mbits, int bias)
{
    if (a == 0.0)
        return 0;
    int e;
    std::frexp(a, &e);
    e -= 1;
    const int emin = 1 - bias;
    if (e < emin)
        e = emin;
    uint32_t r = (uint32_t)std::nearbyint(std::ldexp(a, mbits - e));
    if (e == emin && r < (1u << mbits))
        return r;
    if (r == (2u << mbits)) {
        r >>= 1;
        e += 1;
    }
    return ((uint32_t)(e + bias) << mbits) | (r & ((1u << mbits) - 1u));
}

uint8_t toE4M3(float x)
{
    if (x != x) return 0x7F;
    const uint8_t s = std::signbit(x) ? 0x80 : 0;
    const double a = std::fabs((double)x);
    if (a > 448.0) return s | 0x7E;
    return s | (uint8_t)std::min<uint32_t>(encodeMag(a, 3, 7), 0x7E);
}

uint8_t toE5M2(float x)
{
    if (x != x) return 0x7F;
    const uint8_t s = std::signbit(x) ? 0x80 : 0;
    const double a = std::fabs((double)x);
    if (a > 57344.0) return s | 0x7B;
    return s | (uint8_t)std::min<uint32_t>(encodeMag(a, 2, 15), 0x7B);
}

uint16_t toF16(float x)
{
    const uint16_t s = std::signbit(x) ? 0x8000 : 0;
    if (x != x) return 0x7FFF;
    const double a = std::fabs((double)x);
    if (std::isinf(a)) return s | 0x7C00;
    return s | (uint16_t)std::min<uint32_t>(encodeMag(a, 10, 15), 0x7C00);
}

uint16_t toBF16(float x)
{
    uint32_t b = clpk_f32_bits(x);
    if ((b & 0x7FFFFFFFu) > 0x7F800000u) return 0x7FFF;
    b += 0x7FFFu + ((b >> 16) & 1u);
    return (uint16_t)(b >> 16);
}

double decode(int kind, const uint8_t *t, const uint8_t *sf, int row, int k, int K)
{
    switch (kind) {
    case CLPK_MMA_F16: case CLPK_MMA_F16_F16: return clpk_f16_decode(reinterpret_cast<const uint16_t *>(t)[row * K + k]);
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
        return (double)v * (kind == CLPK_MMA_MXF4 ? clpk_ue8m0_decode(sb) : clpk_e4m3_decode(sb));
    }
    }
}
} // namespace

extern "C" {

const char *clpk_last_error(void) { return g_err; }
const char *clpk_version(void) { return "clpeak-b200 fake shim (CPU test double)"; }

int clpk_device_count(int *count)
{
    *count = fakeDevices();
    return *count > 0 ? CLPK_OK : fail(CLPK_ERR_NO_DEVICE, "no fake devices");
}

int clpk_device_info(int device, clpk_device_info_t *out)
{
    if (device < 0 || device >= fakeDevices()) return fail(CLPK_ERR_BAD_ARG, "bad device");
    std::memset(out, 0, sizeof(*out));
    std::snprintf(out->name, sizeof(out->name), "FAKE B200");
    out->cc_major = 10;
    out->num_sms = 4;
    out->total_mem_bytes = 32ull << 20;
    out->driver_version = 13000;
    out->runtime_version = 12090;
    out->smem_optin_bytes = 232448;
    return CLPK_OK;
}

int clpk_set_device(int device) { g_dev = device; return CLPK_OK; }
int clpk_malloc(void **p, size_t bytes) { *p = std::calloc(1, bytes ? bytes : 1); return *p ? CLPK_OK : fail(CLPK_ERR_CUDA, "oom"); }
int clpk_free(void *p) { std::free(p); return CLPK_OK; }
int clpk_malloc_host(void **p, size_t bytes) { return clpk_malloc(p, bytes); }
int clpk_free_host(void *p) { std::free(p); return CLPK_OK; }
int clpk_memset(void *p, int b, size_t n, void *) { std::memset(p, b, n); return CLPK_OK; }
int clpk_memcpy_h2d(void *d, const void *s, size_t n, void *) { std::memcpy(d, s, n); return CLPK_OK; }
int clpk_memcpy_d2h(void *d, const void *s, size_t n, void *) { std::memcpy(d, s, n); return CLPK_OK; }
int clpk_memcpy_d2d(void *d, const void *s, size_t n, void *) { std::memmove(d, s, n); return CLPK_OK; }
int clpk_stream_create(void **s) { *s = reinterpret_cast<void *>(0x1); return CLPK_OK; }
int clpk_stream_destroy(void *) { return CLPK_OK; }
int clpk_stream_sync(void *) { return CLPK_OK; }

struct FakeEvent { std::chrono::steady_clock::time_point t; };
int clpk_event_create(void **e) { *e = new FakeEvent(); return CLPK_OK; }
int clpk_event_destroy(void *e) { delete static_cast<FakeEvent *>(e); return CLPK_OK; }
int clpk_event_record(void *e, void *) { static_cast<FakeEvent *>(e)->t = std::chrono::steady_clock::now(); return CLPK_OK; }
int clpk_event_sync(void *) { return CLPK_OK; }
int clpk_event_elapsed_ms(void *a, void *b, float *ms)
{
    const auto d = static_cast<FakeEvent *>(b)->t - static_cast<FakeEvent *>(a)->t;
    *ms = std::max(1e-3f, std::chrono::duration<float, std::milli>(d).count());
    return CLPK_OK;
}
int clpk_flush_l2(void *, size_t, void *) { return CLPK_OK; }

int clpk_fill_f32(float *dst, uint64_t n, uint64_t seed, int dist, float mean, float std, void *)
{
    for (uint64_t i = 0; i < n; ++i)
        dst[i] = dist == 0 ? clpk_uniform01(seed, i) : dist == 1 ? clpk_uniform_pm1(seed, i)
                                                                 : std::fmaf(std, clpk_normal01(seed, i), mean);
    return CLPK_OK;
}

int clpk_fill_i8(int8_t *dst, uint64_t n, uint64_t seed, void *)
{
    for (uint64_t i = 0; i < n; ++i) dst[i] = (int8_t)clpk_uniform_i4(seed, i);
    return CLPK_OK;
}

int clpk_convert_f32(void *dst, const float *src, uint64_t n, int dtype, void *)
{
    for (uint64_t i = 0; i < n; ++i) {
        switch (dtype) {
        case CLPK_DT_F16: static_cast<uint16_t *>(dst)[i] = toF16(src[i]); break;
        case CLPK_DT_BF16: static_cast<uint16_t *>(dst)[i] = toBF16(src[i]); break;
        case CLPK_DT_E4M3: static_cast<uint8_t *>(dst)[i] = toE4M3(src[i]); break;
        case CLPK_DT_E5M2: static_cast<uint8_t *>(dst)[i] = toE5M2(src[i]); break;
        case CLPK_DT_I8: static_cast<int8_t *>(dst)[i] = (int8_t)std::max(-128.0, std::min(127.0, std::nearbyint((double)src[i]))); break;
        case CLPK_DT_TF32: {
            uint32_t b = clpk_f32_bits(src[i]);
            if ((b & 0x7F800000u) != 0x7F800000u) b += 0xFFFu + ((b >> 13) & 1u);
            static_cast<uint32_t *>(dst)[i] = b & 0xFFFFE000u;
            break;
        }
        case CLPK_DT_E2M1: {
            uint8_t &byte = static_cast<uint8_t *>(dst)[i / 2];
            const uint8_t nib = clpk_e2m1_encode(src[i]);
            byte = (i & 1) ? (uint8_t)((byte & 0x0F) | (nib << 4)) : nib;
            break;
        }
        default: return fail(CLPK_ERR_BAD_ARG, "dtype");
        }
    }
    return CLPK_OK;
}

int clpk_absmax_f32(float *out, const float *src, uint64_t n, void *)
{
    float m = 0;
    for (uint64_t i = 0; i < n; ++i) m = std::max(m, std::fabs(src[i]));
    *out = m;
    return CLPK_OK;
}

int clpk_quantize_fp4(uint8_t *packed, uint8_t *scales, const float *src, uint64_t rows, uint64_t cols, int dtype,
                      float ts, void *)
{
    const bool mx = dtype == CLPK_DT_MXF4 || dtype == CLPK_DT_MXF4_B64;
    const int blk = dtype == CLPK_DT_MXF4 ? 32 : dtype == CLPK_DT_NVF4 ? 16 : dtype == CLPK_DT_MXF4_B64 ? 64 : 32;
    for (uint64_t b = 0; b < rows * cols / blk; ++b) {
        float v[64], amax = 0;
        for (int i = 0; i < blk; ++i) {
            v[i] = mx ? src[b * blk + i] : src[b * blk + i] / ts;
            amax = std::max(amax, std::fabs(v[i]));
        }
        const uint8_t sb = mx ? clpk_ue8m0_for_absmax(amax) : toE4M3(amax / 6.0f);
        const float sd = mx ? clpk_ue8m0_decode(sb) : clpk_e4m3_decode(sb);
        scales[b] = sb;
        for (int i = 0; i < blk; i += 2) {
            const uint8_t lo = sd > 0 ? clpk_e2m1_encode(v[i] / sd) : 0, hi = sd > 0 ? clpk_e2m1_encode(v[i + 1] / sd) : 0;
            packed[b * (blk / 2) + i / 2] = (uint8_t)(lo | (hi << 4));
        }
    }
    return CLPK_OK;
}

int clpk_global_bandwidth(int width, const float *in, float *out, uint64_t n_floats, void *)
{
    if (n_floats % (256ull * 16 * width)) return fail(CLPK_ERR_BAD_ARG, "ragged");
    const uint64_t outs = n_floats / (16ull * width);
    for (uint64_t o = 0; o < outs; ++o) {
        const uint64_t blk = o / 256, lid = o % 256;
        float lane[4] = {0, 0, 0, 0};
        uint64_t off = blk * 256 * 16 + lid;
        for (int i = 0; i < 16; ++i, off += 256)
            for (int l = 0; l < width; ++l) lane[l] = lane[l] + in[off * width + l];
        float r = lane[0];
        for (int l = 1; l < width; ++l) r = r + lane[l];
        out[o] = r;
    }
    return CLPK_OK;
}

int clpk_stream_read_grid(int variant, int *grid) { *grid = variant == CLPK_STREAM_WIDE ? 4096 : 4; return CLPK_OK; }
int clpk_stream_read(int variant, const void *src, uint64_t n_bytes, uint32_t *parts, void *)
{
    uint32_t x = 0;
    const uint32_t *w = static_cast<const uint32_t *>(src);
    for (uint64_t i = 0; i < n_bytes / 4; ++i) x ^= w[i];
    const int slots = variant == CLPK_STREAM_WIDE ? 4096 : 4;
    for (int i = 1; i < slots; ++i) parts[i] = 0;
    parts[0] = x;
    return CLPK_OK;
}
int clpk_stream_copy(int, void *dst, const void *src, uint64_t n, void *) { std::memcpy(dst, src, n); return CLPK_OK; }
int clpk_stream_triad(int, float *a, const float *b, const float *c, float s, uint64_t n, void *)
{
    for (uint64_t i = 0; i < n; ++i) {
        const float t = s * c[i];
        a[i] = b[i] + t;
    }
    return CLPK_OK;
}
int clpk_stream_status(uint32_t *st, void *) { *st = 0; return CLPK_OK; }
int clpk_stream_checksum_static(const void *src, uint64_t n_bytes, uint32_t grid, uint32_t *out, void *)
{
    if (grid > 4096) return fail(CLPK_ERR_TOO_LARGE, "too many CTAs");
    uint32_t x = 0;
    for (uint64_t i = 0; i < n_bytes / 4; ++i) x ^= static_cast<const uint32_t *>(src)[i];
    *out = x;
    return CLPK_OK;
}

int clpk_compute_sp(float *out, float a, uint32_t grid, void *)
{
    float lane[256];
    for (int l = 0; l < 256; ++l) {
        float x = a;
        const float c = (float)l;
        for (int i = 0; i < 2048; ++i) x = std::fmaf(x, x, c);
        lane[l] = x;
    }
    for (uint64_t i = 0; i < (uint64_t)grid * 256; ++i) out[i] = lane[i % 256];
    return CLPK_OK;
}

int clpk_compute_chain_info(int chain, uint32_t *ops, uint32_t *bytes)
{
    if (chain < 0 || chain >= CLPK_CHAIN_COUNT) return fail(CLPK_ERR_BAD_ARG, "chain");
    if (ops) *ops = chain >= CLPK_CHAIN_INT8_DOT1 ? 8192u : 4096u;
    if (bytes) *bytes = chain == CLPK_CHAIN_DOUBLE ? 8u : 4u;
    return CLPK_OK;
}

int clpk_compute_chain(int chain, void *out, double a, uint32_t grid, void *)
{
    if (chain < 0 || chain >= CLPK_CHAIN_COUNT) return fail(CLPK_ERR_BAD_ARG, "chain");
    uint64_t lane[256];
    for (unsigned l = 0; l < 256; ++l) lane[l] = b200check::typedChainBits(chain, a, l);
    const uint64_t n = (uint64_t)grid * 256;
    if (chain == CLPK_CHAIN_DOUBLE)
        for (uint64_t i = 0; i < n; ++i) static_cast<uint64_t *>(out)[i] = lane[i % 256];
    else
        for (uint64_t i = 0; i < n; ++i) static_cast<uint32_t *>(out)[i] = (uint32_t)lane[i % 256];
    return CLPK_OK;
}

int clpk_local_bandwidth(int width, float *out, uint32_t grid, void *)
{
    if (width != 1 && width != 2 && width != 4) return fail(CLPK_ERR_BAD_ARG, "width");
    for (uint64_t i = 0; i < (uint64_t)grid * 256; ++i) out[i] = b200check::localBandwidthReference(width, i);
    return CLPK_OK;
}

struct FakeImage { uint32_t w, h; uint64_t seed; };

int clpk_image_create(void **image, uint32_t w, uint32_t h, uint64_t seed, void *)
{
    *image = new FakeImage{w, h, seed};
    return CLPK_OK;
}

int clpk_image_bandwidth(void *image, float *out, uint32_t grid, void *)
{
    const FakeImage *im = static_cast<const FakeImage *>(image);
    const uint64_t n = (uint64_t)grid * 256, texels = (uint64_t)im->w * im->h;
    // exact for the threads the host samples (the first and the last 256), zero elsewhere
    for (uint64_t i = 0; i < n; ++i)
        out[i] = (i < 256 || i + 256 >= n) ? b200check::imageBandwidthReference(i, n, texels, im->seed) : 0.0f;
    return CLPK_OK;
}

int clpk_image_bandwidth_tiled(void *image, float *out, uint32_t grid, void *)
{
    const FakeImage *im = static_cast<const FakeImage *>(image);
    const uint64_t n = (uint64_t)grid * 256;
    for (uint64_t i = 0; i < n; ++i)
        out[i] = (i < 256 || i + 256 >= n) ? b200check::imageBandwidthTiledReference(i, im->w, im->h, im->seed) : 0.0f;
    return CLPK_OK;
}

int clpk_image_destroy(void *image)
{
    delete static_cast<FakeImage *>(image);
    return CLPK_OK;
}

int clpk_mad_chain(float *out, uint64_t n_items, uint64_t seed, float y, uint32_t iters, void *)
{
    // exact for the first 4096 work-items (what the host checks), zero beyond
    for (uint64_t i = 0; i < n_items; ++i) {
        if (i >= 4096) { out[i] = 0; continue; }
        float x[4];
        for (int l = 0; l < 4; ++l) x[l] = clpk_uniform_pm1(seed, 4 * i + l);
        for (uint32_t k = 0; k < iters; ++k)
            for (int l = 0; l < 4; ++l) x[l] = std::fmaf(x[l], y, x[l]);
        out[i] = ((x[0] + x[1]) + x[2]) + x[3];
    }
    return CLPK_OK;
}

int clpk_pointer_chase(const uint32_t *next, uint32_t start, uint64_t hops, uint32_t *res, void *)
{
    uint32_t cur = start, x = 0;
    const auto t0 = std::chrono::steady_clock::now();
    for (uint64_t h = 0; h < hops; ++h) { cur = next[cur]; x ^= cur; }
    const uint64_t ns = (uint64_t)std::chrono::duration_cast<std::chrono::nanoseconds>(std::chrono::steady_clock::now() - t0).count() + 1;
    res[0] = cur; res[1] = x; res[2] = (uint32_t)ns; res[3] = (uint32_t)(ns >> 32);
    return CLPK_OK;
}

int clpk_build_chase_cycle(uint32_t *next, uint64_t n, uint64_t seed)
{
    std::vector<uint32_t> order(n);
    for (uint64_t i = 0; i < n; ++i) order[i] = (uint32_t)i;
    for (uint64_t i = n - 1; i > 0; --i) std::swap(order[i], order[clpk_rand64(seed, i) % i]);
    for (uint64_t i = 0; i < n; ++i) next[order[i]] = order[(i + 1) % n];
    return CLPK_OK;
}

int clpk_launch_noop(void *) { return CLPK_OK; }
int clpk_launch_latency(uint32_t, uint32_t, double *mean_us, void *) { *mean_us = 5.0; return CLPK_OK; }
int clpk_graph_launch_latency(uint32_t, uint32_t, uint32_t, double *mean_us, void *) { *mean_us = 1.0; return CLPK_OK; }

int clpk_mma_kind_k(int kind)
{
    switch (kind) {
    case CLPK_MMA_TF32: return 8;
    case CLPK_MMA_F16: case CLPK_MMA_BF16: case CLPK_MMA_F16_F16: return 16;
    case CLPK_MMA_E4M3: case CLPK_MMA_E5M2: case CLPK_MMA_I8: case CLPK_MMA_E2M1: return 32;
    case CLPK_MMA_MXF4: case CLPK_MMA_NVF4: case CLPK_MMA_E4M3_SP: case CLPK_MMA_I8_SP: return 64;
    case CLPK_MMA_MXF4_SP: case CLPK_MMA_NVF4_SP: return 128;
    default: return 0;
    }
}
double clpk_mma_flops_per_instr(int kind) { return 2.0 * 128 * 256 * clpk_mma_kind_k(kind); }

// Sparse kinds on the CPU: expand the compressed A tile through the selector
// nibbles into a dense [128][K] array of doubles, decode B, multiply.
static int fake_sparse_peak(const clpk_mma_peak_args_t *a)
{
    if (!a->d_meta) return fail(CLPK_ERR_BAD_ARG, "sparse kinds need d_meta");
    const int K = clpk_mma_kind_k(a->kind);
    const bool four = K == 128, mx = a->kind == CLPK_MMA_MXF4_SP, integer = a->kind == CLPK_MMA_I8_SP;
    const int nsf = a->kind == CLPK_MMA_NVF4_SP ? 4 : 2, span = K / nsf;
    const uint8_t *A = static_cast<const uint8_t *>(a->d_a), *B = static_cast<const uint8_t *>(a->d_b);
    const uint8_t *M = static_cast<const uint8_t *>(a->d_meta);
    const uint8_t *sfa = static_cast<const uint8_t *>(a->d_sfa), *sfb = static_cast<const uint8_t *>(a->d_sfb);
    auto sf = [&](const uint8_t *t, int row, int k) { return (double)(mx ? clpk_ue8m0_decode(t[row * nsf + k / span]) : clpk_e4m3_decode(t[row * nsf + k / span])); };
    auto nib4 = [](const uint8_t *t, size_t idx) { const uint8_t b = t[idx / 2]; return (uint8_t)((idx & 1) ? b >> 4 : b & 0xF); };
    std::vector<double> da(128 * (size_t)K, 0.0), db(256 * (size_t)K);
    const int unit = four ? 2 : 1;                       // elements per selectable slot
    for (int r = 0; r < 128; ++r)
        for (int grp = 0; grp < K / (4 * unit); ++grp) {
            const uint8_t sel = nib4(M + r * 8, grp);
            const int slot[2] = {sel & 3, sel >> 2};
            for (int which = 0; which < 2; ++which)
                for (int e = 0; e < unit; ++e) {
                    const size_t ci = (size_t)r * (K / 2) + grp * 2 * unit + which * unit + e;
                    const int k = grp * 4 * unit + slot[which] * unit + e;
                    double v;
                    if (four) v = (double)clpk_e2m1_decode(nib4(A, ci)) * sf(sfa, r, k);
                    else if (integer) v = (double)(int8_t)A[ci];
                    else v = (double)clpk_e4m3_decode(A[ci]);
                    da[(size_t)r * K + k] = v;
                }
        }
    for (int r = 0; r < 256; ++r)
        for (int k = 0; k < K; ++k) {
            const size_t i = (size_t)r * K + k;
            db[i] = four ? (double)clpk_e2m1_decode(nib4(B, i)) * sf(sfb, r, k) : integer ? (double)(int8_t)B[i] : (double)clpk_e4m3_decode(B[i]);
        }
    std::vector<uint32_t> tile(128 * 256);
    uint32_t x = 0;
    for (int i = 0; i < 128; ++i)
        for (int j = 0; j < 256; ++j) {
            double p = 0;
            for (int k = 0; k < K; ++k) p += da[(size_t)i * K + k] * db[(size_t)j * K + k];
            const uint32_t w = integer ? (uint32_t)(int32_t)p * a->n_mma : clpk_f32_bits((float)(p * a->n_mma));
            tile[i * 256 + j] = w;
            x ^= w;
        }
    for (uint32_t t = 0; t < a->n_out_tiles; ++t)
        std::memcpy(static_cast<uint32_t *>(a->d_out) + (size_t)t * 128 * 256, tile.data(), tile.size() * 4);
    if (a->d_checksum)
        for (uint32_t c = 0; c < a->grid; ++c) a->d_checksum[c] = x;
    *a->d_status = 0;
    return CLPK_OK;
}

int clpk_mma_peak(const clpk_mma_peak_args_t *a, void *)
{
    const int K = clpk_mma_kind_k(a->kind);
    if (!K) return fail(CLPK_ERR_BAD_ARG, "kind");
    if (a->kind >= CLPK_MMA_E4M3_SP && a->kind <= CLPK_MMA_I8_SP) return fake_sparse_peak(a);
    const uint8_t *A = static_cast<const uint8_t *>(a->d_a), *B = static_cast<const uint8_t *>(a->d_b);
    std::vector<uint32_t> tile(128 * 256);
    uint32_t x = 0;
    for (int i = 0; i < 128; ++i)
        for (int j = 0; j < 256; ++j) {
            double p = 0;
            for (int k = 0; k < K; ++k)
                p += decode(a->kind, A, static_cast<const uint8_t *>(a->d_sfa), i, k, K) *
                     decode(a->kind, B, static_cast<const uint8_t *>(a->d_sfb), j, k, K);
            uint32_t w;
            if (a->kind == CLPK_MMA_I8) w = (uint32_t)(int32_t)p * a->n_mma;
            else if (a->kind == CLPK_MMA_F16_F16) w = clpk_f16_encode((float)(p * a->n_mma));
            else w = clpk_f32_bits((float)(p * a->n_mma));
            tile[i * 256 + j] = w;
            x ^= w;
        }
    for (uint32_t t = 0; t < a->n_out_tiles; ++t)
        std::memcpy(static_cast<uint32_t *>(a->d_out) + (size_t)t * 128 * 256, tile.data(), tile.size() * 4);
    if (a->d_checksum)
        for (uint32_t c = 0; c < a->grid; ++c) a->d_checksum[c] = x;
    *a->d_status = 0;
    return CLPK_OK;
}

int clpk_dmma_peak(const double *a, const double *b, uint32_t n_mma, uint32_t grid, uint32_t n_out_tiles, double *out,
                   uint32_t *checksum, void *)
{
    if (!a || !b || n_out_tiles > grid) return fail(CLPK_ERR_BAD_ARG, "dmma arguments");
    for (uint32_t t = 0; t < n_out_tiles; ++t)
        for (int w = 0; w < CLPK_DMMA_WARPS; ++w)
            for (int r = 0; r < 8; ++r)
                for (int c = 0; c < 8; ++c) {
                    double p = 0, init = 0;
                    for (int k = 0; k < 4; ++k) p += a[r * 4 + k] * b[c * 4 + k];
                    for (int j = 0; j < CLPK_DMMA_CHAINS; ++j) init += w * CLPK_DMMA_CHAINS + j;
                    out[((size_t)t * CLPK_DMMA_WARPS + w) * 64 + r * 8 + c] = init + (double)CLPK_DMMA_CHAINS * n_mma * p;
                }
    if (checksum)
        for (uint32_t c = 0; c < grid; ++c) checksum[c] = 0x1234u;
    return CLPK_OK;
}

int clpk_gemm_last_launch_aligned(void) { return -1; }
int clpk_gemm_last_clock(unsigned long long *c, unsigned long long *n, void *) { *c = 0; *n = 0; return CLPK_OK; }
int clpk_set_tuning(int, int) { return CLPK_OK; }
int clpk_get_tuning(int, int *value) { if (value) *value = -1; return CLPK_OK; }
int clpk_gemm_workspace_bytes(int, uint32_t, uint32_t, uint32_t, size_t *bytes) { *bytes = 0; return CLPK_OK; }
int clpk_gemm(const clpk_gemm_args_t *, void *) { return fail(CLPK_ERR_UNSUPPORTED, "the fake shim has no GEMM"); }
int clpk_gemm_pack_scales(const clpk_gemm_args_t *, void *) { return fail(CLPK_ERR_UNSUPPORTED, "the fake shim has no GEMM"); }

} // extern "C"
