// fp64 tensor-core peak on sm_100a.
//
// tcgen05 has no fp64 kind: the double-precision tensor path of a B200 is the warp-level
// DMMA instruction, mma.sync.aligned.m8n8k4.f64.  This probe takes the place of the
// reference's wmma_fp64 kernel (src/cuda/cuda_kernels/wmma_fp64.cu:15-46; row filled in at
// src/cuda/wmma.cpp:131-138), with two differences: the operands are a seeded tile handed in
// by the caller instead of a constant fill, and the accumulators come back so that the host
// can check them.
//
// Per warp: one A tile [8][4] and one B tile [8][4] (row n holds column n of B, i.e. the
// instruction's ".col" operand) in registers, kDmmaChains independent accumulator tiles.
// Chain j of warp w starts at the value w * kDmmaChains + j in every element, so no two
// chains are the same computation, and runs n_mma dependent instructions D = A*B + D.
// With operands that are multiples of 2^-8 in [-1,1) every product and every partial sum is
// exactly representable (|D| < 2^22 in steps of 2^-16: 38 bits), so the result does not
// depend on the order in which the hardware adds the four products:
//     chain (w, j) ends at  w*kDmmaChains + j + n_mma * (A*B)   exactly.
// Work is counted as the reference counts it: 8*8*4*2 = 512 flop per instruction per warp.
#include "../clpk_internal.h"

namespace clpk {

constexpr int kDmmaWarps = CLPK_DMMA_WARPS;
constexpr int kDmmaChains = CLPK_DMMA_CHAINS;

__device__ __forceinline__ void dmma_m8n8k4(double &d0, double &d1, double a, double b)
{
    asm("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0, %1}, {%2}, {%3}, {%0, %1};"
        : "+d"(d0), "+d"(d1)
        : "d"(a), "d"(b));
}

__global__ void __launch_bounds__(kDmmaWarps * 32)
dmma_peak_kernel(const double *__restrict__ a_tile, const double *__restrict__ b_tile, uint32_t n_mma,
                 uint32_t n_out_tiles, double *__restrict__ out, uint32_t *__restrict__ checksum)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    // fragment layout of m8n8k4: A element (row lane/4, k lane%4); B element (k lane%4, column lane/4);
    // C/D elements (row lane/4, columns 2*(lane%4) and 2*(lane%4)+1)
    const double a = a_tile[(lane >> 2) * 4 + (lane & 3)];
    const double b = b_tile[(lane >> 2) * 4 + (lane & 3)];
    double c[kDmmaChains][2];
#pragma unroll
    for (int j = 0; j < kDmmaChains; j++)
        c[j][0] = c[j][1] = (double)(warp * kDmmaChains + j);

#pragma unroll 1
    for (uint32_t i = 0; i < n_mma; i++) {
#pragma unroll
        for (int j = 0; j < kDmmaChains; j++)
            dmma_m8n8k4(c[j][0], c[j][1], a, b);
    }

    // fold the chains element-wise (exact, see the header comment)
    double s0 = c[0][0], s1 = c[0][1];
#pragma unroll
    for (int j = 1; j < kDmmaChains; j++) {
        s0 += c[j][0];
        s1 += c[j][1];
    }
    if (blockIdx.x < n_out_tiles) {
        double *t = out + ((size_t)blockIdx.x * kDmmaWarps + warp) * 64;
        t[(lane >> 2) * 8 + (lane & 3) * 2] = s0;
        t[(lane >> 2) * 8 + (lane & 3) * 2 + 1] = s1;
    }
    if (checksum) {
        const unsigned long long u0 = (unsigned long long)__double_as_longlong(s0);
        const unsigned long long u1 = (unsigned long long)__double_as_longlong(s1);
        uint32_t x = (uint32_t)u0 ^ (uint32_t)(u0 >> 32) ^ (uint32_t)u1 ^ (uint32_t)(u1 >> 32);
        for (int o = 16; o > 0; o >>= 1)
            x ^= __shfl_xor_sync(0xffffffffu, x, o);
        __shared__ uint32_t wx[kDmmaWarps];
        if (lane == 0)
            wx[warp] = x * (uint32_t)(2 * warp + 1);        // odd multipliers: equal tiles do not cancel
        __syncthreads();
        if (threadIdx.x == 0) {
            uint32_t all = 0;
            for (int w = 0; w < kDmmaWarps; w++)
                all ^= wx[w];
            checksum[blockIdx.x] = all;
        }
    }
}

} // namespace clpk

using namespace clpk;

extern "C" {

int clpk_dmma_peak(const double *d_a, const double *d_b, uint32_t n_mma, uint32_t grid, uint32_t n_out_tiles,
                   double *d_out, uint32_t *d_checksum, void *stream)
{
    int rc = require_sm100();
    if (rc != CLPK_OK)
        return rc;
    CLPK_REQUIRE(d_a && d_b, "NULL tile");
    CLPK_REQUIRE(n_mma >= 1 && grid >= 1, "n_mma and grid must be >= 1");
    CLPK_REQUIRE(n_out_tiles <= grid, "n_out_tiles exceeds grid");
    CLPK_REQUIRE(n_out_tiles == 0 || d_out, "d_out missing");
    dmma_peak_kernel<<<grid, kDmmaWarps * 32, 0, as_stream(stream)>>>(d_a, d_b, n_mma, n_out_tiles, d_out, d_checksum);
    CLPK_LAUNCH_CHECK("dmma_peak");
    return CLPK_OK;
}

} // extern "C"
