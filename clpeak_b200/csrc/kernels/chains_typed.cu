// Shader-core arithmetic chains of the other element types: half, half2, double,
// fp16-in-fp32 ("mixed"), bf16-in-fp32, int32 and the 8-bit dot product with 1, 2, 4
// and 8 independent chains.  They take the place of the reference's compute_hp,
// compute_dp, compute_mp, compute_bf16, compute_int32 and compute_int8_dp kernels
// (src/cuda/cuda_kernels/compute_*.cu; host side src/cuda/compute_float.cpp:30-125,
// src/cuda/compute_int.cpp:10-64) and keep their arithmetic: the recurrence
// x = x*x + c with c = threadIdx.x, the same number of operations per thread
// (4096; 8192 for the dot products) and the same value stored per thread, so a
// host replay of one block's 256 threads checks every launch.
//
// Each chain is one template instantiation of `run<STEPS>()`, a fully unrolled run of
// dependent operations; nothing touches memory until the final store.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "../clpk_internal.h"

namespace clpk {

template <int STEPS>
__device__ __forceinline__ float run_f32(float x, float c)
{
#pragma unroll
    for (int i = 0; i < STEPS; i++)
        x = __fmaf_rn(x, x, c);
    return x;
}

template <int STEPS>
__device__ __forceinline__ __half run_h(__half x, __half c)
{
#pragma unroll
    for (int i = 0; i < STEPS; i++)
        x = __hfma(x, x, c);
    return x;
}

__device__ __forceinline__ uint32_t thread_slot() { return blockIdx.x * 256u + threadIdx.x; }

// two chains of 64 x 16 scalar half FMAs; the store is their half sum, widened
__global__ void __launch_bounds__(256) chain_half_kernel(float *__restrict__ out, float a)
{
    __half x0 = __float2half(a), x1 = __float2half(a + 1.0f);
    const __half c = __float2half((float)threadIdx.x);
#pragma unroll
    for (int i = 0; i < 64; i++) {
        x0 = run_h<16>(x0, c);
        x1 = run_h<16>(x1, c);
    }
    out[thread_slot()] = __half2float(__hadd(x0, x1));
}

// 1024 packed FMAs (two lanes each)
__global__ void __launch_bounds__(256) chain_half2_kernel(float *__restrict__ out, float a)
{
    __half2 x = __float2half2_rn(a);
    const __half2 c = __float2half2_rn((float)threadIdx.x);
#pragma unroll
    for (int i = 0; i < 1024; i++)
        x = __hfma2(x, x, c);
    out[thread_slot()] = __half2float(__low2half(x)) + __half2float(__high2half(x));
}

__global__ void __launch_bounds__(256) chain_double_kernel(double *__restrict__ out, double a)
{
    double x = a;
    const double c = (double)threadIdx.x;
#pragma unroll
    for (int i = 0; i < 2048; i++)
        x = __fma_rn(x, x, c);
    out[thread_slot()] = x;
}

// fp32 FMAs on values that pass through half every 16 steps
__global__ void __launch_bounds__(256) chain_mixed_kernel(float *__restrict__ out, float a)
{
    float x = __half2float(__float2half(a));
    const float c = __half2float(__float2half((float)threadIdx.x));
#pragma unroll
    for (int i = 0; i < 128; i++)
        x = __half2float(__float2half(run_f32<16>(x, c)));
    out[thread_slot()] = x;
}

// fp32 FMAs on values that pass through bfloat16 every 128 steps
__global__ void __launch_bounds__(256) chain_bf16_kernel(float *__restrict__ out, float a)
{
    float x = __bfloat162float(__float2bfloat16(a));
    const float c = __bfloat162float(__float2bfloat16((float)threadIdx.x));
#pragma unroll
    for (int i = 0; i < 16; i++)
        x = __bfloat162float(__float2bfloat16(run_f32<128>(x, c)));
    out[thread_slot()] = x;
}

// wrapping 32-bit multiply-add (unsigned arithmetic: same bits, no signed overflow)
__global__ void __launch_bounds__(256) chain_int32_kernel(int *__restrict__ out, int a)
{
    uint32_t x = (uint32_t)a;
    const uint32_t c = threadIdx.x;
#pragma unroll
    for (int i = 0; i < 2048; i++)
        x = x * x + c;
    out[thread_slot()] = (int)x;
}

// 1024 dot products of four signed bytes, split over CHAINS independent accumulators.
// Chain j starts from y = tid + j and a = tid + offset[j] and repeats a = dp4a(x, y, a);
// y ^= a.  The chains are independent, so the order in which their steps are issued is
// free: here they take turns step by step, BODY dot products per iteration of a rolled
// loop.  The dot-product pipe and the ALU (for the xor) are both close to full, and the
// measured rate moves by a few percent with how ptxas happens to lay the steps out;
// BODY per chain count is the best of 32 / 128 / 512 / 1024 measured on a B200
// (122 / 128 / 125 / 125 TOPS for 1 / 2 / 4 / 8 chains).
template <int CHAINS, int BODY>
__global__ void __launch_bounds__(256) chain_int8_dot_kernel(int *__restrict__ out, int a_arg)
{
    constexpr int kOffsets[4][8] = {{0}, {0, 7}, {0, 7, 13, 19}, {0, 11, 17, 23, 29, 31, 37, 41}};
    constexpr int kRow = CHAINS == 1 ? 0 : CHAINS == 2 ? 1 : CHAINS == 4 ? 2 : 3;
    static_assert(1024 % BODY == 0 && BODY % CHAINS == 0, "BODY must divide 1024 and hold whole rounds");
    const int x = (a_arg & 0xff) | (((a_arg + 1) & 0xff) << 8) | (((a_arg + 2) & 0xff) << 16) |
                  (((a_arg + 3) & 0xff) << 24);
    int y[CHAINS], acc[CHAINS];
#pragma unroll
    for (int j = 0; j < CHAINS; j++) {
        y[j] = (int)threadIdx.x + j;
        acc[j] = (int)threadIdx.x + kOffsets[kRow][j];
    }
#pragma unroll 1
    for (int o = 0; o < 1024 / BODY; o++) {
#pragma unroll
        for (int k = 0; k < BODY / CHAINS; k++) {
#pragma unroll
            for (int j = 0; j < CHAINS; j++) {
                acc[j] = __dp4a(x, y[j], acc[j]);
                y[j] ^= acc[j];
            }
        }
    }
    uint32_t sum = 0;
#pragma unroll
    for (int j = 0; j < CHAINS; j++)
        sum += (uint32_t)acc[j];
    out[thread_slot()] = (int)sum;
}

} // namespace clpk

using namespace clpk;

extern "C" {

int clpk_compute_chain_info(int chain, uint32_t *ops_per_thread, uint32_t *out_elem_bytes)
{
    CLPK_REQUIRE(chain >= 0 && chain < CLPK_CHAIN_COUNT, "unknown chain %d", chain);
    if (ops_per_thread)
        *ops_per_thread = chain >= CLPK_CHAIN_INT8_DOT1 ? 8192u : 4096u;
    if (out_elem_bytes)
        *out_elem_bytes = chain == CLPK_CHAIN_DOUBLE ? 8u : 4u;
    return CLPK_OK;
}

int clpk_compute_chain(int chain, void *d_out, double a, uint32_t grid, void *stream)
{
    int rc = require_sm100();
    if (rc != CLPK_OK)
        return rc;
    CLPK_REQUIRE(chain >= 0 && chain < CLPK_CHAIN_COUNT, "unknown chain %d", chain);
    CLPK_REQUIRE(d_out && grid > 0, "bad arguments");
    cudaStream_t s = as_stream(stream);
    float *of = static_cast<float *>(d_out);
    int *oi = static_cast<int *>(d_out);
    switch (chain) {
    case CLPK_CHAIN_HALF:      chain_half_kernel<<<grid, 256, 0, s>>>(of, (float)a); break;
    case CLPK_CHAIN_HALF2:     chain_half2_kernel<<<grid, 256, 0, s>>>(of, (float)a); break;
    case CLPK_CHAIN_DOUBLE:    chain_double_kernel<<<grid, 256, 0, s>>>(static_cast<double *>(d_out), a); break;
    case CLPK_CHAIN_MIXED:     chain_mixed_kernel<<<grid, 256, 0, s>>>(of, (float)a); break;
    case CLPK_CHAIN_BF16:      chain_bf16_kernel<<<grid, 256, 0, s>>>(of, (float)a); break;
    case CLPK_CHAIN_INT32:     chain_int32_kernel<<<grid, 256, 0, s>>>(oi, (int)a); break;
    case CLPK_CHAIN_INT8_DOT1: chain_int8_dot_kernel<1, 1024><<<grid, 256, 0, s>>>(oi, (int)a); break;
    case CLPK_CHAIN_INT8_DOT2: chain_int8_dot_kernel<2, 128><<<grid, 256, 0, s>>>(oi, (int)a); break;
    case CLPK_CHAIN_INT8_DOT4: chain_int8_dot_kernel<4, 1024><<<grid, 256, 0, s>>>(oi, (int)a); break;
    default:                   chain_int8_dot_kernel<8, 32><<<grid, 256, 0, s>>>(oi, (int)a); break;
    }
    CLPK_LAUNCH_CHECK("compute_chain");
    return CLPK_OK;
}

} // extern "C"
