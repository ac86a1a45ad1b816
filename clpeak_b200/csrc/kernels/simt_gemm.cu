// The two GEMM rows that have no tcgen05 kind: fp32 on the CUDA cores and fp64 on the
// warp-level DMMA path.  They take the place of the reference's cuBLASLt "fp32" and
// "fp64" rows (src/cuda/cuda_blas.cpp:567-581) behind the same clpk_gemm entry point:
// C[M][N] = alpha * A[M][K] * B[N][K]^T, both operands K-contiguous, C row-major in the
// operand type.
//
// fp32 (sgemm_kernel).  128 x 128 x 16 tile per CTA of 128 threads = 4 warps in a 2 x 2
// grid, two CTAs per SM, 8 rows x 16 columns of outputs per thread.  The multiply is
// sm_100's packed fma.rn.f32x2 (two FMAs per issued instruction) on accumulator pairs of
// neighbouring columns, the row value duplicated into a fresh register pair just before
// its eight FMAs.  Which shape the packed FMA likes was measured from registers alone: 8
// rows x 8 pairs with that duplication runs at 71 of 74 TFLOPS with 8 warps per SM, 16
// rows x 4 pairs at 51, pairs over two neighbouring k (no duplication at all) at 52 --
// the operand pairs collide in the register banks.  Operands are transposed into shared
// memory ([k][row]) so that both fragments are 128-bit loads: global -> staging buffer by
// asynchronous 16-byte copies two k blocks ahead, staging -> registers -> tile by the
// thread that copied them, one barrier per k block.  Fragment loads are laid out for two
// passes of the shared-memory data pipe per 128-bit load (see the kernel).  Bound: the
// fp32 pipe, 128 FMA / clock / SM (B200: 148 SMs x 128 x 2 x 1.965 GHz = 74.4 TFLOPS).
// Measured 62.6 TFLOPS at 8192^3 (0.84 of the pipe, 0.95 of cuBLAS) and 60.8 at 4096^3
// (1.07 of cuBLAS: 1024 tiles are 3.5 waves of 296 CTAs, and a CTA alone on its SM runs
// twice as fast).  The same loop runs at 68.4 without the transposition, 65.2 without the
// fragment loads and 69.6 with neither; moving the transposition under the multiplies
// (with or without a branch) and 128-bit tile stores changed nothing; leaving A as it lies
// in memory (fragments of four k per row, only B transposed) ran at 53.5.  Earlier shapes:
// 256 threads x (8 x 8) with the next k block held in registers across the multiply,
// 54.0 (the warps stood at the tile stores waiting for the global loads); the same through
// the staging buffer, 58.9.
//
// fp64 (dgemm_kernel).  128 x 64 x 16 tile per CTA of 128 threads = 4 warps in a 2 x 2
// grid, two CTAs per SM, 64 x 32 outputs per warp = 8 x 4 m8n8k4 accumulator tiles (128
// registers of accumulators per thread).  Operands go global -> shared with cp.async (16 bytes), three
// stages; rows are padded to 20 doubles so that the fragment reads (lane -> row lane/4,
// k lane%4) fall in 16 distinct 8-byte banks per half warp.  Bound: the DMMA pipe, 64
// fp64 FMA / clock / SM, the same rate as the scalar DFMA pipe (37.2 TFLOPS at 1.965 GHz).
//
// Both take any M, N > 0 and any K that keeps operand rows 16-byte aligned (a multiple of 4
// floats, 2 doubles): a second instantiation of each kernel zero-fills the chunks a tile
// reaches beyond A or B (cp.async with a source size of 0) and skips the stores beyond C;
// whole tiles and k blocks take the instantiation without the checks.
//
// CTAs walk C in groups of 16 tile rows so that the operand panels a wave of CTAs needs
// stay in L2.  Work 2*M*N*K flop; minimum HBM bytes (M*K + N*K + M*N) * element.
#include "../clpk_internal.h"

namespace clpk {

constexpr int kSimtTile = 128;
constexpr int kSimtBK = 16;
constexpr int kRasterGroup = 16;

// blockIdx.x -> (tile row, tile column), column-major inside groups of kRasterGroup tile rows
__device__ __forceinline__ void raster(uint32_t tiles_m, uint32_t tiles_n, uint32_t *tm, uint32_t *tn)
{
    const uint32_t per_group = kRasterGroup * tiles_n;
    const uint32_t g = blockIdx.x / per_group, r = blockIdx.x % per_group;
    const uint32_t rows = min((uint32_t)kRasterGroup, tiles_m - g * kRasterGroup);
    *tm = g * kRasterGroup + r % rows;
    *tn = r / rows;
}

// ---------------------------------------------------------------------------------------------
// fp32
// ---------------------------------------------------------------------------------------------

__device__ __forceinline__ unsigned long long pack2(float lo, float hi)
{
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}

__device__ __forceinline__ float2 unpack2(unsigned long long v)
{
    float2 r;
    asm("mov.b64 {%0, %1}, %2;" : "=f"(r.x), "=f"(r.y) : "l"(v));
    return r;
}

// d = a * b + d on two packed fp32 lanes, each rounded to nearest even like fmaf
__device__ __forceinline__ void ffma2(unsigned long long &d, unsigned long long a, unsigned long long b)
{
    asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(d) : "l"(a), "l"(b));
}

constexpr int kSgemmLd = kSimtTile + 4;               // floats per k row of a shared tile
constexpr int kSgemmThreads = 128;
constexpr int kSgemmChunks = 2 * kSimtTile * kSimtBK / 4 / kSgemmThreads;      // 16-byte chunks per thread and k block
constexpr size_t kSgemmTileFloats = (size_t)kSimtBK * kSgemmLd;                // one operand, one buffer: [k][row]
constexpr size_t kSgemmStagingFloats = kSgemmChunks * 4 * (size_t)kSgemmThreads;
constexpr size_t kSgemmSmemBytes = (4 * kSgemmTileFloats + 2 * kSgemmStagingFloats) * sizeof(float);

__device__ __forceinline__ void cp_async_16(void *dst_shared, const void *src)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst_shared)), "l"(src) : "memory");
}

// the same copy, or 16 bytes of zeros when the chunk lies outside the operand (nothing is read then)
__device__ __forceinline__ void cp_async_16_or_zeros(void *dst_shared, const void *src, bool inside)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"((uint32_t)__cvta_generic_to_shared(dst_shared)), "l"(src),
                 "r"(inside ? 16u : 0u)
                 : "memory");
}

// RAGGED: M, N need not be multiples of the tile nor K of the k block (K a multiple of 4, so that rows stay 16-byte
// aligned): chunks outside the operands arrive as zeros, stores outside C are skipped.
template <bool RAGGED>
__global__ void __launch_bounds__(kSgemmThreads, 2)
sgemm_kernel(const float *__restrict__ A, const float *__restrict__ B, float *__restrict__ C, uint32_t M, uint32_t N,
             uint32_t K, float alpha)
{
    extern __shared__ __align__(16) float ssm[];
    float *const tiles = ssm;                                   // [buffer][A, B][k][kSgemmLd]
    float *const staging = ssm + 4 * kSgemmTileFloats;          // [buffer][chunk][thread] of float4
    uint32_t tm, tn;
    raster((M + kSimtTile - 1) / kSimtTile, (N + kSimtTile - 1) / kSimtTile, &tm, &tn);
    // Four warps in a 2 x 2 grid, 64 x 64 outputs per warp, a warp 8 (rows) x 4 (columns) threads, 8 rows x 16
    // columns per thread as 4 x 4 blocks.  A 128-bit shared-memory load takes two passes of the data pipe per warp
    // when every group of four consecutive lanes asks for at most two different 16-byte words, and four passes
    // otherwise (measured with a one-warp probe: lane / 2, lane / 4 and lane % 2 cost two passes, lane % 4 and
    // lane % 8 four).  So lane bits 0 and 2 pick the column block and bits 1, 3, 4 the row block: inside a group of
    // four lanes both fragments have two distinct addresses.
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int lx = (lane & 1) | ((lane >> 1) & 2), ly = ((lane >> 1) & 1) | ((lane >> 2) & 6);
    const int fa = (warp >> 1) * 64 + ly * 4, fb = (warp & 1) * 64 + lx * 4;

    // Operands travel global -> staging (asynchronous 16-byte copies, two k blocks ahead) -> registers -> tile
    // (transposed: [row][k] in memory, [k][row] in the tile).  Every thread moves the same chunks through both
    // hops -- rows lrow + 32 c of A and of B, floats lk .. lk + 3 of the k block -- so only its own copies have to
    // have landed before it transposes, and nothing read from global memory is held in registers across the
    // multiply (with the loads going straight to registers the warps stood at the tile stores waiting for them:
    // 53 against 64 TFLOPS for the same loop without the operand traffic).
    const int lrow = tid >> 2, lk = (tid & 3) * 4;
    const float *srcA = A + ((size_t)tm * kSimtTile + lrow) * K + lk, *srcB = B + ((size_t)tn * kSimtTile + lrow) * K + lk;
    auto fetch = [&](uint32_t kb) {                              // k block kb into staging buffer kb % 2
        float *st = staging + (kb & 1) * kSgemmStagingFloats + tid * 4;
#pragma unroll
        for (int c = 0; c < 4; c++) {
            if (RAGGED) {
                const bool in_k = kb * kSimtBK + lk < K;
                const bool in_a = in_k && tm * kSimtTile + lrow + 32 * c < M, in_b = in_k && tn * kSimtTile + lrow + 32 * c < N;
                cp_async_16_or_zeros(st + c * 4 * kSgemmThreads, in_a ? srcA + (size_t)c * 32 * K + (size_t)kb * kSimtBK : A, in_a);
                cp_async_16_or_zeros(st + (4 + c) * 4 * kSgemmThreads, in_b ? srcB + (size_t)c * 32 * K + (size_t)kb * kSimtBK : B, in_b);
            } else {
                cp_async_16(st + c * 4 * kSgemmThreads, srcA + (size_t)c * 32 * K + (size_t)kb * kSimtBK);
                cp_async_16(st + (4 + c) * 4 * kSgemmThreads, srcB + (size_t)c * 32 * K + (size_t)kb * kSimtBK);
            }
        }
    };
    auto transpose = [&](uint32_t kb) {                          // staging buffer kb % 2 into tile buffer kb % 2
        const float *st = staging + (kb & 1) * kSgemmStagingFloats + tid * 4;
        float *sA = tiles + (kb & 1) * 2 * kSgemmTileFloats, *sB = sA + kSgemmTileFloats;
#pragma unroll
        for (int c = 0; c < 8; c++) {
            const float4 v = *reinterpret_cast<const float4 *>(st + c * 4 * kSgemmThreads);
            // k rows 8..15 keep their columns with bit 3 flipped: a warp stores 8 consecutive rows for four k
            // (lk = 0, 4, 8, 12), and 8 k rows of 132 floats are a multiple of 32 banks apart
            float *dst = (c < 4 ? sA : sB) + lk * kSgemmLd + ((lrow + 32 * (c & 3)) ^ (lk & 8));
            dst[0] = v.x; dst[kSgemmLd] = v.y; dst[2 * kSgemmLd] = v.z; dst[3 * kSgemmLd] = v.w;
        }
    };

    // Accumulators as pairs of neighbouring columns: sm_100's packed fma.rn.f32x2 does two FMAs per issued
    // instruction with the rounding of two scalar FMAs.  8 rows x 8 pairs with the row value duplicated into a
    // fresh register pair just before its eight FMAs runs at 71 of 74 TFLOPS from registers alone with 8 warps per
    // SM; 16 rows x 4 pairs at 51 (register-bank conflicts between the operand pairs).
    unsigned long long acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; i++)
#pragma unroll
        for (int j = 0; j < 8; j++)
            acc[i][j] = 0ull;

    const uint32_t nk = (K + kSimtBK - 1) / kSimtBK;
    fetch(0);
    asm volatile("cp.async.commit_group;" ::: "memory");
    if (nk > 1)
        fetch(1);
    asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group 1;" ::: "memory");
    transpose(0);
    __syncthreads();
    for (uint32_t kb = 0; kb < nk; kb++) {
        // staging buffer kb % 2 was emptied into the tile before the last barrier: refill it two k blocks ahead
        if (kb + 2 < nk)
            fetch(kb + 2);
        asm volatile("cp.async.commit_group;" ::: "memory");
        const float *sA = tiles + (kb & 1) * 2 * kSgemmTileFloats, *sB = sA + kSgemmTileFloats;
#pragma unroll
        for (int k = 0; k < kSimtBK; k++) {
            const int ca = fa ^ (k & 8), cb = fb ^ (k & 8);
            float a[8];
            unsigned long long b[8];
#pragma unroll
            for (int q = 0; q < 2; q++) {
                const float4 v = *reinterpret_cast<const float4 *>(sA + k * kSgemmLd + ca + 32 * q);
                a[4 * q] = v.x; a[4 * q + 1] = v.y; a[4 * q + 2] = v.z; a[4 * q + 3] = v.w;
            }
#pragma unroll
            for (int h = 0; h < 4; h++) {
                const float4 v = *reinterpret_cast<const float4 *>(sB + k * kSgemmLd + cb + 16 * h);
                b[2 * h] = pack2(v.x, v.y);
                b[2 * h + 1] = pack2(v.z, v.w);
            }
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const unsigned long long aa = pack2(a[i], a[i]);
#pragma unroll
                for (int j = 0; j < 8; j++)
                    ffma2(acc[i][j], aa, b[j]);
            }
        }
        if (kb + 1 < nk) {
            asm volatile("cp.async.wait_group 1;" ::: "memory");      // k block kb + 1 is in staging (kb + 2 may still fly)
            transpose(kb + 1);
            __syncthreads();
        }
    }

    float *gC = C + (size_t)tm * kSimtTile * N + (size_t)tn * kSimtTile;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const int r = fa + 32 * (i >> 2) + (i & 3);
#pragma unroll
        for (int h = 0; h < 4; h++) {
            const float2 lo = unpack2(acc[i][2 * h]), hi = unpack2(acc[i][2 * h + 1]);
            const float4 v = make_float4(alpha * lo.x, alpha * lo.y, alpha * hi.x, alpha * hi.y);
            if (!RAGGED) {
                *reinterpret_cast<float4 *>(gC + (size_t)r * N + fb + 16 * h) = v;
            } else if (tm * kSimtTile + r < M) {
                const uint32_t col = tn * kSimtTile + fb + 16 * h;
                float *dst = gC + (size_t)r * N + fb + 16 * h;
                if ((N & 3) == 0 && col < N) {
                    *reinterpret_cast<float4 *>(dst) = v;
                } else {
                    const float e[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                    for (int t = 0; t < 4; t++)
                        if (col + t < N)
                            dst[t] = e[t];
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// fp64
// ---------------------------------------------------------------------------------------------

constexpr int kDgemmLd = kSimtBK + 4;                    // doubles per row of a shared tile (160 bytes)
constexpr int kDgemmStages = 3;
// CN = columns of C per CTA.  64: four warps and two CTAs per SM, whose barriers and pipeline fills overlap each
// other; with 128 (eight warps, one CTA per SM) the DMMA pipe idled at every CTA-wide barrier (87 % busy in ncu).
template <int CN> struct Dgemm {
    static constexpr int threads = 2 * CN;
    static constexpr size_t stage_doubles = (size_t)(kSimtTile + CN) * kDgemmLd;
    static constexpr size_t smem_bytes = kDgemmStages * stage_doubles * sizeof(double);
};

__device__ __forceinline__ void dmma_m8n8k4(double &d0, double &d1, double a, double b)
{
    asm("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0, %1}, {%2}, {%3}, {%0, %1};"
        : "+d"(d0), "+d"(d1)
        : "d"(a), "d"(b));
}

template <int CN, bool RAGGED>
__global__ void __launch_bounds__(Dgemm<CN>::threads, 128 / CN)
dgemm_kernel(const double *__restrict__ A, const double *__restrict__ B, double *__restrict__ C, uint32_t M, uint32_t N,
             uint32_t K, double alpha)
{
    extern __shared__ __align__(16) double dsm[];
    constexpr int kThreads = Dgemm<CN>::threads;
    constexpr size_t kDgemmStageDoubles = Dgemm<CN>::stage_doubles;
    uint32_t tm, tn;
    raster((M + kSimtTile - 1) / kSimtTile, (N + CN - 1) / CN, &tm, &tn);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    constexpr int kWarpsN = CN / 32;
    const int wm = (warp / kWarpsN) * 64, wn = (warp % kWarpsN) * 32;   // this warp's 64 x 32 corner inside the tile
    const double *gA = A + (size_t)tm * kSimtTile * K, *gB = B + (size_t)tn * CN * K;

    // one stage = A tile [128][kDgemmLd] then B tile [CN][kDgemmLd]; 16-byte chunks, 8 per row
    auto load_stage = [&](int stage, uint32_t k0) {
        double *sa = dsm + (size_t)stage * kDgemmStageDoubles, *sb = sa + (size_t)kSimtTile * kDgemmLd;
#pragma unroll
        for (int i = 0; i < kSimtTile * 8 / kThreads; i++) {
            const int c = tid + kThreads * i, r = c >> 3, kc = (c & 7) * 2;
            if (RAGGED) {
                const bool inside = tm * kSimtTile + r < M && k0 + kc < K;
                cp_async_16_or_zeros(sa + r * kDgemmLd + kc, inside ? gA + (size_t)r * K + k0 + kc : A, inside);
            } else {
                cp_async_16(sa + r * kDgemmLd + kc, gA + (size_t)r * K + k0 + kc);
            }
        }
#pragma unroll
        for (int i = 0; i < CN * 8 / kThreads; i++) {
            const int c = tid + kThreads * i, r = c >> 3, kc = (c & 7) * 2;
            if (RAGGED) {
                const bool inside = tn * CN + r < N && k0 + kc < K;
                cp_async_16_or_zeros(sb + r * kDgemmLd + kc, inside ? gB + (size_t)r * K + k0 + kc : B, inside);
            } else {
                cp_async_16(sb + r * kDgemmLd + kc, gB + (size_t)r * K + k0 + kc);
            }
        }
    };

    double acc[8][4][2];
#pragma unroll
    for (int i = 0; i < 8; i++)
#pragma unroll
        for (int j = 0; j < 4; j++)
            acc[i][j][0] = acc[i][j][1] = 0.0;

    const uint32_t nk = (K + kSimtBK - 1) / kSimtBK;
#pragma unroll
    for (int s = 0; s < kDgemmStages - 1; s++) {
        if ((uint32_t)s < nk)
            load_stage(s, s * kSimtBK);
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    const int fr = lane >> 2, fk = lane & 3;                        // fragment row (or column of B) and k of this lane
    for (uint32_t kb = 0; kb < nk; kb++) {
        asm volatile("cp.async.wait_group %0;" ::"n"(kDgemmStages - 2) : "memory");
        __syncthreads();                                            // stage kb has landed; stage kb-1 is free for reuse
        if (kb + kDgemmStages - 1 < nk)
            load_stage((kb + kDgemmStages - 1) % kDgemmStages, (kb + kDgemmStages - 1) * kSimtBK);
        asm volatile("cp.async.commit_group;" ::: "memory");
        const double *sa = dsm + (size_t)(kb % kDgemmStages) * kDgemmStageDoubles, *sb = sa + (size_t)kSimtTile * kDgemmLd;
#pragma unroll
        for (int k4 = 0; k4 < kSimtBK; k4 += 4) {
            double a[8], b[4];
#pragma unroll
            for (int i = 0; i < 8; i++)
                a[i] = sa[(wm + 8 * i + fr) * kDgemmLd + k4 + fk];
#pragma unroll
            for (int j = 0; j < 4; j++)
                b[j] = sb[(wn + 8 * j + fr) * kDgemmLd + k4 + fk];
#pragma unroll
            for (int i = 0; i < 8; i++)
#pragma unroll
                for (int j = 0; j < 4; j++)
                    dmma_m8n8k4(acc[i][j][0], acc[i][j][1], a[i], b[j]);
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");

    // accumulator tile (i, j): this lane holds row lane/4, columns 2*(lane%4) and the next one
    double *gC = C + ((size_t)tm * kSimtTile + wm) * N + (size_t)tn * CN + wn;
#pragma unroll
    for (int i = 0; i < 8; i++)
#pragma unroll
        for (int j = 0; j < 4; j++)
        {
            double *dst = gC + (size_t)(8 * i + fr) * N + 8 * j + 2 * fk;
            const double2 v = make_double2(alpha * acc[i][j][0], alpha * acc[i][j][1]);
            if (!RAGGED) {
                *reinterpret_cast<double2 *>(dst) = v;
            } else if (tm * kSimtTile + wm + 8 * i + fr < M) {
                const uint32_t col = tn * CN + wn + 8 * j + 2 * fk;
                if ((N & 1) == 0 && col < N) {
                    *reinterpret_cast<double2 *>(dst) = v;
                } else {
                    if (col < N)
                        dst[0] = v.x;
                    if (col + 1 < N)
                        dst[1] = v.y;
                }
            }
        }
}

int launch_simt_gemm(int dtype, const void *a, const void *b, void *c, uint32_t m, uint32_t n, uint32_t k, float alpha,
                     cudaStream_t s)
{
    CLPK_REQUIRE(m > 0 && n > 0 && k > 0, "M, N and K must be positive");
    const uint32_t k_unit = dtype == CLPK_DT_F32 ? 4 : 2;            // elements per 16 bytes: operand rows stay aligned
    CLPK_REQUIRE(k % k_unit == 0, "K = %u: a row of A and B must be a multiple of 16 bytes", k);
    CLPK_REQUIRE(((uintptr_t)a % 16) == 0 && ((uintptr_t)b % 16) == 0 && ((uintptr_t)c % 16) == 0, "operands must be 16-byte aligned");
    const uint32_t tile_n = dtype == CLPK_DT_F32 ? kSimtTile : 64;
    const uint64_t tiles = (uint64_t)((m + kSimtTile - 1) / kSimtTile) * ((n + tile_n - 1) / tile_n);
    CLPK_REQUIRE(tiles <= 0x3FFFFFFFull, "too many tiles");
    // whole tiles and whole k blocks take the kernel without the bounds checks
    const bool ragged = m % kSimtTile != 0 || n % tile_n != 0 || k % kSimtBK != 0;
    if (dtype == CLPK_DT_F32) {
        auto kernel = ragged ? sgemm_kernel<true> : sgemm_kernel<false>;
        CLPK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSgemmSmemBytes));
        kernel<<<(unsigned)tiles, kSgemmThreads, kSgemmSmemBytes, s>>>(static_cast<const float *>(a), static_cast<const float *>(b),
                                                                      static_cast<float *>(c), m, n, k, alpha);
        CLPK_LAUNCH_CHECK("sgemm");
    } else {
        // 128 x 64 CTA tiles: 34.2-34.5 TFLOPS at 4096^3 / 8192^3 against 31.9-32.1 with 128 x 128 tiles of 8 warps
        auto kernel = ragged ? dgemm_kernel<64, true> : dgemm_kernel<64, false>;
        CLPK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Dgemm<64>::smem_bytes));
        kernel<<<(unsigned)tiles, Dgemm<64>::threads, Dgemm<64>::smem_bytes, s>>>(
            static_cast<const double *>(a), static_cast<const double *>(b), static_cast<double *>(c), m, n, k, (double)alpha);
        CLPK_LAUNCH_CHECK("dgemm");
    }
    return CLPK_OK;
}

} // namespace clpk
