// Seeded operand generation, format conversion and block-scaled FP4
// quantisation.  These are set-up kernels: they run outside every timed
// region, so they are written for determinism, not speed.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include "../clpk_internal.h"
#include "../clpk_rng.h"
#include "../clpk_formats.h"

namespace clpk {

__global__ void fill_f32_kernel(float *dst, uint64_t n, uint64_t seed, int dist, float mean,
                                float stdv)
{
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        float v;
        if (dist == CLPK_DIST_UNIFORM01)
            v = clpk_uniform01(seed, i);
        else if (dist == CLPK_DIST_UNIFORM_PM1)
            v = clpk_uniform_pm1(seed, i);
        else
            v = __fmaf_rn(stdv, clpk_normal01(seed, i), mean);
        dst[i] = v;
    }
}

__global__ void fill_i8_kernel(int8_t *dst, uint64_t n, uint64_t seed)
{
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        dst[i] = (int8_t)clpk_uniform_i4(seed, i);
}

__global__ void convert_kernel(void *dst, const float *src, uint64_t n, int dtype)
{
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const float x = src[i];
        switch (dtype) {
        case CLPK_DT_F16:
            reinterpret_cast<__half *>(dst)[i] = __float2half_rn(x);
            break;
        case CLPK_DT_BF16:
            reinterpret_cast<__nv_bfloat16 *>(dst)[i] = __float2bfloat16_rn(x);
            break;
        case CLPK_DT_E4M3:
            reinterpret_cast<uint8_t *>(dst)[i] = __nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3);
            break;
        case CLPK_DT_E5M2:
            reinterpret_cast<uint8_t *>(dst)[i] = __nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E5M2);
            break;
        case CLPK_DT_TF32: {
            // nearest even at bit 13 in integer arithmetic (infinities and NaNs keep their class)
            uint32_t b = __float_as_uint(x);
            if ((b & 0x7F800000u) != 0x7F800000u)
                b += 0xFFFu + ((b >> 13) & 1u);
            reinterpret_cast<uint32_t *>(dst)[i] = b & 0xFFFFE000u;
            break;
        }
        case CLPK_DT_F64:
            reinterpret_cast<double *>(dst)[i] = (double)x;
            break;
        case CLPK_DT_I8: {
            int v = __float2int_rn(x);
            v = v < -128 ? -128 : (v > 127 ? 127 : v);
            reinterpret_cast<int8_t *>(dst)[i] = (int8_t)v;
            break;
        }
        default:
            break;
        }
    }
}

__global__ void convert_e2m1_kernel(uint8_t *dst, const float *src, uint64_t n_pairs)
{
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_pairs; i += stride)
        dst[i] = (uint8_t)(clpk_e2m1_encode(src[2 * i]) | (clpk_e2m1_encode(src[2 * i + 1]) << 4));
}

__global__ void absmax_kernel(float *out, const float *src, uint64_t n)
{
    float m = 0.0f;
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        m = fmaxf(m, fabsf(src[i]));
    for (int o = 16; o > 0; o >>= 1)
        m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    // |x| >= 0, so the float ordering equals the ordering of the bit patterns.
    if ((threadIdx.x & 31) == 0)
        atomicMax(reinterpret_cast<unsigned int *>(out), __float_as_uint(m));
}

// One thread per scale block of BLOCK elements; UE8M0 selects the scale format
// (power-of-two MX scale) against ue4m3 (NVFP4 scale, after the tensor scale).
template <int BLOCK, bool UE8M0>
__global__ void quantize_fp4_kernel(uint8_t *packed, uint8_t *scales, const float *src,
                                    uint64_t n_blocks, float tensor_scale)
{
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t b = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; b < n_blocks; b += stride) {
        const float *x = src + b * BLOCK;
        float v[BLOCK];
        float amax = 0.0f;
#pragma unroll
        for (int i = 0; i < BLOCK; i++) {
            v[i] = UE8M0 ? x[i] : __fdiv_rn(x[i], tensor_scale);
            amax = fmaxf(amax, fabsf(v[i]));
        }
        uint8_t sbyte;
        float sdec;
        if (UE8M0) {
            sbyte = clpk_ue8m0_for_absmax(amax);
            sdec = clpk_ue8m0_decode(sbyte);
        } else {
            sbyte = __nv_cvt_float_to_fp8(__fdiv_rn(amax, 6.0f), __NV_SATFINITE, __NV_E4M3);
            sdec = clpk_e4m3_decode(sbyte);
        }
        scales[b] = sbyte;
        uint8_t *p = packed + b * (BLOCK / 2);
#pragma unroll
        for (int i = 0; i < BLOCK; i += 2) {
            uint8_t lo = 0, hi = 0;
            if (sdec > 0.0f) {
                lo = clpk_e2m1_encode(__fdiv_rn(v[i], sdec));
                hi = clpk_e2m1_encode(__fdiv_rn(v[i + 1], sdec));
            }
            p[i / 2] = (uint8_t)(lo | (hi << 4));
        }
    }
}

__global__ void flush_kernel(uint4 *p, uint64_t n16, uint32_t tag)
{
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += stride)
        p[i] = make_uint4(tag, tag, tag, tag);
}

static int fill_grid()
{
    int sms = num_sms();
    return sms > 0 ? sms * 8 : 1024;
}

} // namespace clpk

using namespace clpk;

extern "C" {

int clpk_fill_f32(float *d_dst, uint64_t n, uint64_t seed, int dist, float mean, float std,
                  void *stream)
{
    CLPK_REQUIRE(d_dst || n == 0, "d_dst is NULL");
    CLPK_REQUIRE(dist >= 0 && dist <= 2, "unknown distribution %d", dist);
    if (n == 0)
        return CLPK_OK;
    fill_f32_kernel<<<fill_grid(), 256, 0, as_stream(stream)>>>(d_dst, n, seed, dist, mean, std);
    CLPK_LAUNCH_CHECK("fill_f32");
    return CLPK_OK;
}

int clpk_fill_i8(int8_t *d_dst, uint64_t n, uint64_t seed, void *stream)
{
    CLPK_REQUIRE(d_dst || n == 0, "d_dst is NULL");
    if (n == 0)
        return CLPK_OK;
    fill_i8_kernel<<<fill_grid(), 256, 0, as_stream(stream)>>>(d_dst, n, seed);
    CLPK_LAUNCH_CHECK("fill_i8");
    return CLPK_OK;
}

int clpk_convert_f32(void *d_dst, const float *d_src, uint64_t n, int dtype, void *stream)
{
    CLPK_REQUIRE((d_dst && d_src) || n == 0, "NULL buffer");
    CLPK_REQUIRE(dtype == CLPK_DT_F16 || dtype == CLPK_DT_BF16 || dtype == CLPK_DT_E4M3 ||
                     dtype == CLPK_DT_E5M2 || dtype == CLPK_DT_I8 || dtype == CLPK_DT_TF32 || dtype == CLPK_DT_E2M1 ||
                     dtype == CLPK_DT_F64,
                 "clpk_convert_f32: dtype %d has no plain conversion", dtype);
    if (n == 0)
        return CLPK_OK;
    if (dtype == CLPK_DT_E2M1) {
        CLPK_REQUIRE(n % 2 == 0, "E2M1 packs two elements per byte: n (%llu) must be even", (unsigned long long)n);
        convert_e2m1_kernel<<<fill_grid(), 256, 0, as_stream(stream)>>>(static_cast<uint8_t *>(d_dst), d_src, n / 2);
        CLPK_LAUNCH_CHECK("convert_e2m1");
        return CLPK_OK;
    }
    convert_kernel<<<fill_grid(), 256, 0, as_stream(stream)>>>(d_dst, d_src, n, dtype);
    CLPK_LAUNCH_CHECK("convert");
    return CLPK_OK;
}

int clpk_absmax_f32(float *d_absmax, const float *d_src, uint64_t n, void *stream)
{
    CLPK_REQUIRE(d_absmax, "d_absmax is NULL");
    CLPK_CUDA(cudaMemsetAsync(d_absmax, 0, sizeof(float), as_stream(stream)));
    if (n == 0)
        return CLPK_OK;
    CLPK_REQUIRE(d_src, "d_src is NULL");
    absmax_kernel<<<fill_grid(), 256, 0, as_stream(stream)>>>(d_absmax, d_src, n);
    CLPK_LAUNCH_CHECK("absmax");
    return CLPK_OK;
}

int clpk_quantize_fp4(uint8_t *d_packed, uint8_t *d_scales, const float *d_src, uint64_t rows,
                      uint64_t cols, int dtype, float tensor_scale, void *stream)
{
    CLPK_REQUIRE(d_packed && d_scales && d_src, "NULL buffer");
    const bool mx = (dtype == CLPK_DT_MXF4 || dtype == CLPK_DT_MXF4_B64);
    CLPK_REQUIRE(mx || dtype == CLPK_DT_NVF4 || dtype == CLPK_DT_NVF4_B32, "dtype must be an MXF4 or NVF4 variant");
    CLPK_REQUIRE(cols % 64 == 0, "cols (%llu) must be a multiple of 64", (unsigned long long)cols);
    CLPK_REQUIRE(mx || tensor_scale > 0.0f, "tensor_scale must be positive");
    const uint64_t n = rows * cols;
    if (n == 0)
        return CLPK_OK;
    const int g = fill_grid();
    cudaStream_t s = as_stream(stream);
    switch (dtype) {
    case CLPK_DT_MXF4:     quantize_fp4_kernel<32, true><<<g, 128, 0, s>>>(d_packed, d_scales, d_src, n / 32, 1.0f); break;
    case CLPK_DT_MXF4_B64: quantize_fp4_kernel<64, true><<<g, 128, 0, s>>>(d_packed, d_scales, d_src, n / 64, 1.0f); break;
    case CLPK_DT_NVF4:     quantize_fp4_kernel<16, false><<<g, 128, 0, s>>>(d_packed, d_scales, d_src, n / 16, tensor_scale); break;
    default:               quantize_fp4_kernel<32, false><<<g, 128, 0, s>>>(d_packed, d_scales, d_src, n / 32, tensor_scale); break;
    }
    CLPK_LAUNCH_CHECK("quantize_fp4");
    return CLPK_OK;
}

int clpk_flush_l2(void *d_scratch, size_t bytes, void *stream)
{
    CLPK_REQUIRE(d_scratch, "d_scratch is NULL");
    static unsigned tag = 0;
    flush_kernel<<<fill_grid(), 256, 0, as_stream(stream)>>>(reinterpret_cast<uint4 *>(d_scratch),
                                                            bytes / 16, ++tag);
    CLPK_LAUNCH_CHECK("flush_l2");
    return CLPK_OK;
}

} // extern "C"
