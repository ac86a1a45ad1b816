// Tensor-core peak probes on tcgen05.mma.
//
// One CTA = 128 threads.  It stages an A tile [128][K] and a B tile [256][K]
// (K contiguous) into shared memory, allocates tensor memory for a 128x256
// 32-bit accumulator and lets one thread issue n_mma instructions of shape
// M128 N256 K that all accumulate into that tile; a tcgen05.commit arrives on
// an mbarrier when the last one has retired.  The four warps then read the
// accumulator back with tcgen05.ld (warp w owns TMEM lanes 32w..32w+31),
// XOR it into a per-CTA checksum and, for the first n_out_tiles CTAs, store it.
//
// Shared-memory operand layout (no swizzle, K-major): every dense kind has
// 32 bytes of K per row per instruction (16 x 16-bit, 32 x 8-bit, 64 x 4-bit),
// i.e. two 16-byte chunks.  An 8-row x 16-byte "core matrix" is 128
// contiguous bytes; the two K chunks of a row group sit side by side (leading
// offset 128 B) and row groups follow each other (stride offset 256 B):
//     byte(r, kc) = (r / 8) * 256 + kc * 128 + (r % 8) * 16
//
// Block-scaled kinds keep their scale factors in tensor memory: row r of A has
// one 32-bit word (up to four 8-bit factors along K) at lane r % 32, column
// r / 32 of the scale area, replicated in all four 32-lane quarters; B's 256
// rows take 8 columns the same way.  The probes write them with tcgen05.st.
//
// kind::tf32 reads 32-bit words (K = 8 per instruction) and ignores the low 13 mantissa
// bits; the fp16-accumulate variant of kind::f16 keeps a 16-bit accumulator in the low
// half of each 32-bit tensor-memory cell.
//
// Residency: dense kinds take 256 TMEM columns, so two CTAs fit one SM; the
// launch asks for enough dynamic shared memory that a third never becomes
// resident (tcgen05.alloc would otherwise block on it).  Kinds with scale
// factors or metadata take all 512 columns: one CTA per SM.
#include <cstdlib>

#include "../clpk_internal.h"
#include "../clpk_ptx.cuh"

namespace clpk {

constexpr int kTileM = 128;
constexpr int kTileN = 256;
constexpr int kRowBytes = 32;                       // K bytes per row per instruction
constexpr int kATileBytes = kTileM * kRowBytes;     // 4 KiB
constexpr int kBTileBytes = kTileN * kRowBytes;     // 8 KiB

struct PeakParams {
    const uint8_t *a;
    const uint8_t *b;
    const uint8_t *sfa;
    const uint8_t *sfb;
    const uint8_t *meta;
    uint32_t n_mma;
    uint32_t n_out_tiles;
    uint32_t *out;
    uint32_t *checksum;
    uint32_t *status;
    unsigned long long *clock;  // optional: CTA 0 stores {SM cycles, nanoseconds} from its first issue to its last retire
    uint32_t lone_lane;         // 1: the issue loop runs in one thread (the form kept for comparison)
};

// Copy a [rows][32 B] row-major tile into the core-matrix layout.
__device__ __forceinline__ void stage_tile(uint8_t *smem_tile, const uint8_t *g, int rows)
{
    const int chunks = rows * 2;
    for (int i = threadIdx.x; i < chunks; i += blockDim.x) {
        const int r = i >> 1, kc = i & 1;
        const uint4 v = *reinterpret_cast<const uint4 *>(g + (size_t)r * kRowBytes + kc * 16);
        *reinterpret_cast<uint4 *>(smem_tile + (r >> 3) * 256 + kc * 128 + (r & 7) * 16) = v;
    }
}

// Unscaled 4-bit operands of kind::f8f6f4: the input tile is [rows][32] e2m1 packed two per
// byte (16 bytes per row); in shared memory every 16 elements (8 bytes) sit at the start of
// a 16-byte slot whose other half is padding, so a row again takes two 16-byte chunks.
__device__ __forceinline__ void stage_tile_fp4_padded(uint8_t *smem_tile, const uint8_t *g, int rows)
{
    const int chunks = rows * 2;
    for (int i = threadIdx.x; i < chunks; i += blockDim.x) {
        const int r = i >> 1, kc = i & 1;
        const uint2 v = *reinterpret_cast<const uint2 *>(g + (size_t)r * 16 + kc * 8);
        *reinterpret_cast<uint4 *>(smem_tile + (r >> 3) * 256 + kc * 128 + (r & 7) * 16) = make_uint4(v.x, v.y, 0u, 0u);
    }
}

template <int KIND>
struct KindTraits;
template <> struct KindTraits<CLPK_MMA_TF32>    { static constexpr bool scaled = false; static constexpr int sf_per_row = 0; };
template <> struct KindTraits<CLPK_MMA_F16_F16> { static constexpr bool scaled = false; static constexpr int sf_per_row = 0; };
template <> struct KindTraits<CLPK_MMA_E2M1>    { static constexpr bool scaled = false; static constexpr int sf_per_row = 0; };
template <> struct KindTraits<CLPK_MMA_F16>  { static constexpr bool scaled = false; static constexpr int sf_per_row = 0; };
template <> struct KindTraits<CLPK_MMA_BF16> { static constexpr bool scaled = false; static constexpr int sf_per_row = 0; };
template <> struct KindTraits<CLPK_MMA_E4M3> { static constexpr bool scaled = false; static constexpr int sf_per_row = 0; };
template <> struct KindTraits<CLPK_MMA_E5M2> { static constexpr bool scaled = false; static constexpr int sf_per_row = 0; };
template <> struct KindTraits<CLPK_MMA_I8>   { static constexpr bool scaled = false; static constexpr int sf_per_row = 0; };
template <> struct KindTraits<CLPK_MMA_MXF4> { static constexpr bool scaled = true;  static constexpr int sf_per_row = 2; };
template <> struct KindTraits<CLPK_MMA_NVF4> { static constexpr bool scaled = true;  static constexpr int sf_per_row = 4; };

// PAIR: the cta_group::2 form.  The two CTAs of a cluster hold the same A tile and one
// half of B each (B rows [128r, 128r + 128) in CTA r); one instruction of shape M256 N256
// fills both CTAs' 128 x 256 accumulators with the same A.B^T tile a lone CTA computes.
// Per flop it reads a third less shared memory (B once per pair), which under the power
// cap is worth a few per cent of clock.
template <int KIND, bool PAIR>
__device__ __forceinline__ void issue_mma(uint32_t d, uint64_t ad, uint64_t bd, uint32_t sfa,
                                          uint32_t sfb, uint32_t acc)
{
    constexpr uint32_t M = PAIR ? 256 : kTileM;
    if constexpr (KIND == CLPK_MMA_F16 || KIND == CLPK_MMA_BF16 || KIND == CLPK_MMA_F16_F16) {
        const uint32_t fmt = KIND == CLPK_MMA_BF16 ? kFmtBF16 : kFmtF16;
        const uint32_t idesc = make_idesc(M, kTileN, fmt, fmt, KIND == CLPK_MMA_F16_F16 ? kAccF16 : kAccF32);
        if constexpr (PAIR) mma2_f16_ss(d, ad, bd, idesc, acc); else mma_f16_ss(d, ad, bd, idesc, acc);
    } else if constexpr (KIND == CLPK_MMA_E4M3 || KIND == CLPK_MMA_E5M2 || KIND == CLPK_MMA_E2M1) {
        const uint32_t fmt = KIND == CLPK_MMA_E4M3 ? kFmtE4M3 : KIND == CLPK_MMA_E5M2 ? kFmtE5M2 : kFmtE2M1x8;
        const uint32_t idesc = make_idesc(M, kTileN, fmt, fmt, kAccF32);
        if constexpr (PAIR) mma2_f8f6f4_ss(d, ad, bd, idesc, acc); else mma_f8f6f4_ss(d, ad, bd, idesc, acc);
    } else if constexpr (KIND == CLPK_MMA_I8) {
        const uint32_t idesc = make_idesc(M, kTileN, kFmtS8, kFmtS8, kAccS32);
        if constexpr (PAIR) mma2_i8_ss(d, ad, bd, idesc, acc); else mma_i8_ss(d, ad, bd, idesc, acc);
    } else if constexpr (KIND == CLPK_MMA_TF32) {
        const uint32_t idesc = make_idesc(M, kTileN, kFmtTF32, kFmtTF32, kAccF32);
        if constexpr (PAIR) mma2_tf32_ss(d, ad, bd, idesc, acc); else mma_tf32_ss(d, ad, bd, idesc, acc);
    } else if constexpr (KIND == CLPK_MMA_MXF4) {
        const uint32_t idesc = make_idesc_block_scaled(M, kTileN, kFmtE2M1, kFmtE2M1, /*ue8m0*/ 1, 0, 0);
        if constexpr (PAIR) mma2_mxf4_bs(d, ad, bd, idesc, sfa, sfb, acc); else mma_mxf4_bs(d, ad, bd, idesc, sfa, sfb, acc);
    } else if constexpr (KIND == CLPK_MMA_NVF4) {
        const uint32_t idesc = make_idesc_block_scaled(M, kTileN, kFmtE2M1, kFmtE2M1, /*ue4m3*/ 0, 0, 0);
        if constexpr (PAIR) mma2_nvf4_bs(d, ad, bd, idesc, sfa, sfb, acc); else mma_nvf4_bs(d, ad, bd, idesc, sfa, sfb, acc);
    }
}

template <int KIND, bool PAIR>
__global__ void __launch_bounds__(128) mma_peak_kernel(PeakParams p)
{
    using T = KindTraits<KIND>;
    constexpr uint32_t kCols = T::scaled ? 512u : 256u;
    constexpr uint32_t kSfaCol = 256, kSfbCol = 260;
    constexpr int kGroup = PAIR ? 2 : 1;
    constexpr int kBRows = PAIR ? kTileN / 2 : kTileN;          // rows of B this CTA stages

    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t *sA = smem;
    uint8_t *sB = smem + kATileBytes;
    uint64_t *bar = reinterpret_cast<uint64_t *>(smem + kATileBytes + kBTileBytes);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bar + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = PAIR ? cluster_ctarank() : 0u;
    const uint8_t *b_rows = p.b + (size_t)rank * kBRows * (KIND == CLPK_MMA_E2M1 ? 16 : kRowBytes);

    if constexpr (KIND == CLPK_MMA_E2M1) {
        stage_tile_fp4_padded(sA, p.a, kTileM);
        stage_tile_fp4_padded(sB, b_rows, kBRows);
    } else {
        stage_tile(sA, p.a, kTileM);
        stage_tile(sB, b_rows, kBRows);
    }
    if (threadIdx.x == 0) {
        mbar_init(bar, 1);
        mbar_fence_init();
    }
    fence_proxy_async_smem();
    if (warp == 0) {
        __syncwarp();
        tmem_alloc<kGroup>(tmem_slot, kCols);
    }
    tc_fence_before_sync();
    __syncthreads();
    if constexpr (PAIR)
        cluster_sync();                 // both CTAs' tiles, barriers and tensor memory are in place
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;

    if constexpr (T::scaled) {
        // Scale factors: one 32-bit word per row, factors along K in byte order.
        const uint32_t lane_base = tmem + ((uint32_t)(warp * 32) << 16);
        for (int c = 0; c < 4; c++) {
            const int r = c * 32 + lane;
            uint32_t w = 0;
            for (int k = 0; k < T::sf_per_row; k++)
                w |= (uint32_t)p.sfa[r * T::sf_per_row + k] << (8 * k);
            tmem_st_32x32b_x1(lane_base + kSfaCol + c, w);
        }
        for (int c = 0; c < 8; c++) {
            const int r = c * 32 + lane;
            uint32_t w = 0;
            for (int k = 0; k < T::sf_per_row; k++)
                w |= (uint32_t)p.sfb[r * T::sf_per_row + k] << (8 * k);
            tmem_st_32x32b_x1(lane_base + kSfbCol + c, w);
        }
        tmem_st_wait();
        tc_fence_before_sync();
        __syncthreads();
        if constexpr (PAIR)
            cluster_sync();
        tc_fence_after_sync();
    }

    // The issue loop runs in the whole of warp 0 and one elected lane issues: inside `if (lane == 0)`
    // every tcgen05.mma costs its thread about as long as the tensor core needs for it, so a lone
    // issuer cannot run ahead of the pipe; as a convergent warp an issue takes a quarter of that.
    unsigned long long c0 = 0, t0 = 0;
    if (warp == 0 && rank == 0) {
        const uint64_t ad = make_smem_desc(smem_u32(sA), 128, 256, kSwizzleNone);
        const uint64_t bd = make_smem_desc(smem_u32(sB), 128, 256, kSwizzleNone);
        const uint32_t sfa = tmem + kSfaCol, sfb = tmem + kSfbCol;
        c0 = clock64();
        t0 = globaltimer_ns();
        if (p.lone_lane) {
            if (lane == 0) {
                issue_mma<KIND, PAIR>(tmem, ad, bd, sfa, sfb, 0u);
                for (uint32_t i = 1; i < p.n_mma; i++)
                    issue_mma<KIND, PAIR>(tmem, ad, bd, sfa, sfb, 1u);
                if constexpr (PAIR) tc_commit_pair(bar, 3); else tc_commit(bar);
            }
        } else {
            if (elect_one())
                issue_mma<KIND, PAIR>(tmem, ad, bd, sfa, sfb, 0u);
            for (uint32_t i = 1; i < p.n_mma; i++)
                if (elect_one())
                    issue_mma<KIND, PAIR>(tmem, ad, bd, sfa, sfb, 1u);
            if (elect_one()) {
                if constexpr (PAIR) tc_commit_pair(bar, 3); else tc_commit(bar);
            }
        }
    }
    __syncwarp();

    // The verdict must be uniform across the CTA: the tcgen05.ld below is a
    // warp-aligned instruction and the checksum uses a CTA barrier.
    const int done = __syncthreads_and(mbar_wait(bar, 0) ? 1 : 0);
    tc_fence_after_sync();
    if (p.clock && blockIdx.x == 0 && threadIdx.x == 0) {
        p.clock[0] = clock64() - c0;
        p.clock[1] = globaltimer_ns() - t0;
    }
    if (!done && threadIdx.x == 0)
        atomicCAS(p.status, 0u, 0x100u + (uint32_t)KIND);

    uint32_t x = 0;
    if (done) {
        const int row = warp * 32 + lane;
        uint32_t *out_row = (blockIdx.x < p.n_out_tiles)
                                ? p.out + ((size_t)blockIdx.x * kTileM + row) * kTileN
                                : nullptr;
        for (int c = 0; c < kTileN / 32; c++) {
            uint32_t r[32];
            tmem_ld_32x32b_x32(tmem + ((uint32_t)(warp * 32) << 16) + c * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; i++)
                x ^= r[i];
            if (out_row) {
#pragma unroll
                for (int i = 0; i < 32; i += 4)
                    *reinterpret_cast<uint4 *>(out_row + c * 32 + i) =
                        make_uint4(r[i], r[i + 1], r[i + 2], r[i + 3]);
            }
        }
    }
    __shared__ uint32_t wx[4];
    for (int o = 16; o > 0; o >>= 1)
        x ^= __shfl_xor_sync(0xffffffffu, x, o);
    if (lane == 0)
        wx[warp] = x;
    __syncthreads();
    if (done && p.checksum && threadIdx.x == 0)
        p.checksum[blockIdx.x] = wx[0] ^ wx[1] ^ wx[2] ^ wx[3];

    tc_fence_before_sync();
    __syncthreads();
    if constexpr (PAIR)
        cluster_sync();                 // the peer's shared memory and barrier stay valid until both are done
    if (warp == 0)
        tmem_dealloc<kGroup>(tmem, kCols);
}


// ---------------------------------------------------------------------------------
// 2:4 structured-sparse kinds (tcgen05.mma.sp)
// ---------------------------------------------------------------------------------
//
// A arrives compressed: [128][K/2] elements = 32 bytes per row, staged exactly like
// a dense A tile.  B is dense over the logical K = 64 (8-bit kinds): 64 bytes per
// row, staged in the 128-byte-swizzle K-major layout (row pitch 128 B, 8-row atoms
// of 1024 B, 16-byte chunk c of row r stored at chunk c ^ (r % 8)); the instruction
// reads the first 64 bytes of each row.  The metadata -- one 4-bit selector per
// group of four logical K positions, low 2 bits = position of the first kept
// element, high 2 bits = position of the second -- lives in tensor memory:
// row r in lane r, its K/8 selector bytes in K order in consecutive columns.

constexpr int kSpBRowBytes = 64;
constexpr int kSpBPitch = 128;
constexpr int kSpBTileBytes = kTileN * kSpBPitch;   // 32 KiB

__device__ __forceinline__ void stage_tile_sw128(uint8_t *smem_tile, const uint8_t *g, int rows, int row_bytes)
{
    const int chunks_per_row = row_bytes / 16;
    for (int i = threadIdx.x; i < rows * chunks_per_row; i += blockDim.x) {
        const int r = i / chunks_per_row, c = i % chunks_per_row;
        const uint4 v = *reinterpret_cast<const uint4 *>(g + (size_t)r * row_bytes + c * 16);
        *reinterpret_cast<uint4 *>(smem_tile + r * kSpBPitch + ((c ^ (r & 7)) * 16)) = v;
    }
}

// PAIR: two CTAs run one cta_group::2 instruction (M = 256).  Both stage the same compressed A
// tile and metadata, each half of B's rows, so each ends with the same 128 x 256 result as a
// lone CTA.  It matters here more than for the dense kinds: a lone CTA reads 4 KiB of A and
// 16 KiB of B from shared memory per instruction, 160 cycles at 128 bytes per cycle against the
// 128 cycles the tensor core needs (measured: 163), a pair 4 + 8 KiB each.
template <int KIND, bool PAIR>
__global__ void __launch_bounds__(128) mma_peak_sparse_kernel(PeakParams p, uint32_t meta_cols)
{
    constexpr int kGroup = PAIR ? 2 : 1;
    constexpr int kBRows = PAIR ? kTileN / 2 : kTileN;          // rows of B this CTA stages
    constexpr uint32_t kM = PAIR ? 256 : kTileM;
    const uint32_t rank = PAIR ? cluster_ctarank() : 0u;
    constexpr uint32_t kCols = 512;
    constexpr uint32_t kMetaCol = 256, kSpSfaCol = 260, kSpSfbCol = 264;
    constexpr bool kScaled = (KIND == CLPK_MMA_MXF4_SP || KIND == CLPK_MMA_NVF4_SP);
    constexpr int kSfPerRow = (KIND == CLPK_MMA_NVF4_SP) ? 4 : 2;

    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t *sA = smem;                                 // 4 KiB, core-matrix layout
    uint8_t *sB = smem + 4096;                          // 32 KiB, 1024-aligned
    uint64_t *bar = reinterpret_cast<uint64_t *>(smem + 4096 + kSpBTileBytes);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bar + 1);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    stage_tile(sA, p.a, kTileM);
    stage_tile_sw128(sB, p.b + (size_t)rank * kBRows * kSpBRowBytes, kBRows, kSpBRowBytes);
    if (threadIdx.x == 0) {
        mbar_init(bar, 1);
        mbar_fence_init();
    }
    fence_proxy_async_smem();
    if (warp == 0) {
        __syncwarp();
        tmem_alloc<kGroup>(tmem_slot, kCols);
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;

    // metadata image: word (row, c) -> lane row, column kMetaCol + c
    {
        const uint32_t *meta = reinterpret_cast<const uint32_t *>(p.meta);
        const int row = warp * 32 + lane;
        const uint32_t lane_base = tmem + ((uint32_t)(warp * 32) << 16);
        for (uint32_t c = 0; c < meta_cols; c++)
            tmem_st_32x32b_x1(lane_base + kMetaCol + c, meta[row * meta_cols + c]);
        if constexpr (kScaled) {
            // scale factors as in the dense block-scaled kinds: row r -> lane r % 32, column r / 32
            for (int c = 0; c < 4; c++) {
                uint32_t w = 0;
                for (int k = 0; k < kSfPerRow; k++)
                    w |= (uint32_t)p.sfa[(c * 32 + lane) * kSfPerRow + k] << (8 * k);
                tmem_st_32x32b_x1(lane_base + kSpSfaCol + c, w);
            }
            for (int c = 0; c < 8; c++) {
                uint32_t w = 0;
                for (int k = 0; k < kSfPerRow; k++)
                    w |= (uint32_t)p.sfb[(c * 32 + lane) * kSfPerRow + k] << (8 * k);
                tmem_st_32x32b_x1(lane_base + kSpSfbCol + c, w);
            }
        }
        tmem_st_wait();
        tc_fence_before_sync();
        __syncthreads();
        if constexpr (PAIR)
            cluster_sync();             // both CTAs' tiles, metadata, barriers and tensor memory are in place
        tc_fence_after_sync();
    }

    unsigned long long c0 = 0, t0 = 0;
    if (warp == 0 && rank == 0) {
        const uint64_t ad = make_smem_desc(smem_u32(sA), 128, 256, kSwizzleNone);
        const uint64_t bd = make_smem_desc(smem_u32(sB), 16, 1024, kSwizzle128B);
        c0 = clock64();
        t0 = globaltimer_ns();
        uint32_t idesc;
        if constexpr (KIND == CLPK_MMA_I8_SP)
            idesc = make_idesc(kM, kTileN, kFmtS8, kFmtS8, kAccS32, true);
        else if constexpr (KIND == CLPK_MMA_E4M3_SP)
            idesc = make_idesc(kM, kTileN, kFmtE4M3, kFmtE4M3, kAccF32, true);
        else
            idesc = make_idesc_block_scaled(kM, kTileN, kFmtE2M1, kFmtE2M1, KIND == CLPK_MMA_MXF4_SP ? 1u : 0u, 0, 0, true);
        for (uint32_t i = 0; i < p.n_mma; i++) {
            const uint32_t acc = i ? 1u : 0u, meta_t = tmem + kMetaCol, sfa_t = tmem + kSpSfaCol, sfb_t = tmem + kSpSfbCol;
            // whole warp in the loop, one lane issues (see the dense kernel); lone_lane keeps lane 0 alone
            if (!(p.lone_lane ? lane == 0 : elect_one() != 0))
                continue;
            if constexpr (KIND == CLPK_MMA_I8_SP) {
                if constexpr (PAIR) mma2_i8_sp(tmem, ad, bd, idesc, meta_t, acc); else mma_i8_sp(tmem, ad, bd, idesc, meta_t, acc);
            } else if constexpr (KIND == CLPK_MMA_E4M3_SP) {
                if constexpr (PAIR) mma2_f8f6f4_sp(tmem, ad, bd, idesc, meta_t, acc); else mma_f8f6f4_sp(tmem, ad, bd, idesc, meta_t, acc);
            } else if constexpr (KIND == CLPK_MMA_MXF4_SP) {
                if constexpr (PAIR) mma2_mxf4_sp_bs(tmem, ad, bd, idesc, meta_t, sfa_t, sfb_t, acc);
                else mma_mxf4_sp_bs(tmem, ad, bd, idesc, meta_t, sfa_t, sfb_t, acc);
            } else {
                if constexpr (PAIR) mma2_nvf4_sp_bs(tmem, ad, bd, idesc, meta_t, sfa_t, sfb_t, acc);
                else mma_nvf4_sp_bs(tmem, ad, bd, idesc, meta_t, sfa_t, sfb_t, acc);
            }
        }
        if (p.lone_lane ? lane == 0 : elect_one() != 0) {
            if constexpr (PAIR) tc_commit_pair(bar, 3); else tc_commit(bar);
        }
    }
    __syncwarp();

    const int done = __syncthreads_and(mbar_wait(bar, 0) ? 1 : 0);
    tc_fence_after_sync();
    if (p.clock && blockIdx.x == 0 && threadIdx.x == 0) {
        p.clock[0] = clock64() - c0;
        p.clock[1] = globaltimer_ns() - t0;
    }
    if (!done && threadIdx.x == 0)
        atomicCAS(p.status, 0u, 0x100u + (uint32_t)KIND);

    uint32_t x = 0;
    if (done) {
        const int row = warp * 32 + lane;
        uint32_t *out_row = (blockIdx.x < p.n_out_tiles) ? p.out + ((size_t)blockIdx.x * kTileM + row) * kTileN : nullptr;
        for (int c = 0; c < kTileN / 32; c++) {
            uint32_t r[32];
            tmem_ld_32x32b_x32(tmem + ((uint32_t)(warp * 32) << 16) + c * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; i++)
                x ^= r[i];
            if (out_row) {
#pragma unroll
                for (int i = 0; i < 32; i += 4)
                    *reinterpret_cast<uint4 *>(out_row + c * 32 + i) = make_uint4(r[i], r[i + 1], r[i + 2], r[i + 3]);
            }
        }
    }
    __shared__ uint32_t wx[4];
    for (int o = 16; o > 0; o >>= 1)
        x ^= __shfl_xor_sync(0xffffffffu, x, o);
    if (lane == 0)
        wx[warp] = x;
    __syncthreads();
    if (done && p.checksum && threadIdx.x == 0)
        p.checksum[blockIdx.x] = wx[0] ^ wx[1] ^ wx[2] ^ wx[3];

    tc_fence_before_sync();
    __syncthreads();
    if constexpr (PAIR)
        cluster_sync();                 // the peer's shared memory and barrier stay valid until both are done
    if (warp == 0)
        tmem_dealloc<kGroup>(tmem, kCols);
}

template <int KIND>
static int launch_peak_sparse(const PeakParams &p, uint32_t grid, uint32_t meta_cols, cudaStream_t s)
{
    const size_t smem = (size_t)(smem_optin_bytes() * 3 / 5);      // one CTA per SM (512 TMEM columns)
    // CTA pairs by default (a lone CTA is bound by shared-memory reads); the MMA_PAIR knob overrides.
    bool pair = true;
    if (const int t = tuning(CLPK_TUNE_MMA_PAIR); t >= 0)
        pair = t == 1;
    if (grid % 2 == 0 && pair) {
        CLPK_CUDA(cudaFuncSetAttribute(mma_peak_sparse_kernel<KIND, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(grid);
        cfg.blockDim = dim3(128);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = s;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        const cudaError_t e = cudaLaunchKernelEx(&cfg, mma_peak_sparse_kernel<KIND, true>, p, meta_cols);
        if (e != cudaSuccess)
            return cuda_fail(e, "launch mma_peak_sparse (pairs)");
        return CLPK_OK;
    }
    CLPK_CUDA(cudaFuncSetAttribute(mma_peak_sparse_kernel<KIND, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    mma_peak_sparse_kernel<KIND, false><<<grid, 128, smem, s>>>(p, meta_cols);
    CLPK_LAUNCH_CHECK("mma_peak_sparse");
    return CLPK_OK;
}

struct KindInfo {
    int k;              // logical K per instruction
    bool scaled;
    bool sparse;
};

static bool kind_info(int kind, KindInfo *ki)
{
    switch (kind) {
    case CLPK_MMA_F16:     *ki = {16, false, false}; return true;
    case CLPK_MMA_BF16:    *ki = {16, false, false}; return true;
    case CLPK_MMA_E4M3:    *ki = {32, false, false}; return true;
    case CLPK_MMA_E5M2:    *ki = {32, false, false}; return true;
    case CLPK_MMA_I8:      *ki = {32, false, false}; return true;
    case CLPK_MMA_TF32:    *ki = {8, false, false};  return true;
    case CLPK_MMA_F16_F16: *ki = {16, false, false}; return true;
    case CLPK_MMA_E2M1:    *ki = {32, false, false}; return true;
    case CLPK_MMA_MXF4:    *ki = {64, true, false};  return true;
    case CLPK_MMA_NVF4:    *ki = {64, true, false};  return true;
    case CLPK_MMA_E4M3_SP: *ki = {64, false, true};  return true;
    case CLPK_MMA_I8_SP:   *ki = {64, false, true};  return true;
    case CLPK_MMA_MXF4_SP: *ki = {128, true, true};  return true;
    case CLPK_MMA_NVF4_SP: *ki = {128, true, true};  return true;
    default: return false;
    }
}

template <int KIND>
static int launch_peak(const PeakParams &p, uint32_t grid, cudaStream_t s)
{
    // Dense: ~100 KiB so that exactly two CTAs fit one SM; scaled: one CTA.
    const int optin = smem_optin_bytes();
    const size_t smem = KindTraits<KIND>::scaled ? (size_t)(optin * 3 / 5) : (size_t)(optin * 2 / 5);
    // CTA pairs (cta_group::2) where they measured faster on B200 -- int8 +1.5..4 %, MXFP4 / NVFP4 +2..4 %;
    // fp16 / bf16 / fp8 lose 4..7 % as pairs and stay solo.  The MMA_PAIR knob (0 / 1) overrides for every kind.
    bool pair = KIND == CLPK_MMA_I8 || KIND == CLPK_MMA_MXF4 || KIND == CLPK_MMA_NVF4;
    if (const int t = tuning(CLPK_TUNE_MMA_PAIR); t >= 0)
        pair = t == 1;
    if (grid % 2 == 0 && pair) {
        CLPK_CUDA(cudaFuncSetAttribute(mma_peak_kernel<KIND, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(grid);
        cfg.blockDim = dim3(128);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = s;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        const cudaError_t e = cudaLaunchKernelEx(&cfg, mma_peak_kernel<KIND, true>, p);
        if (e != cudaSuccess)
            return cuda_fail(e, "launch mma_peak (pairs)");
        return CLPK_OK;
    }
    CLPK_CUDA(cudaFuncSetAttribute(mma_peak_kernel<KIND, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   (int)smem));
    mma_peak_kernel<KIND, false><<<grid, 128, smem, s>>>(p);
    CLPK_LAUNCH_CHECK("mma_peak");
    return CLPK_OK;
}

} // namespace clpk

using namespace clpk;

extern "C" {

int clpk_mma_kind_k(int kind)
{
    KindInfo ki;
    return kind_info(kind, &ki) ? ki.k : 0;
}

double clpk_mma_flops_per_instr(int kind)
{
    KindInfo ki;
    if (!kind_info(kind, &ki))
        return 0.0;
    return 2.0 * kTileM * kTileN * (double)ki.k;
}

int clpk_mma_peak(const clpk_mma_peak_args_t *a, void *stream)
{
    int rc = require_sm100();
    if (rc != CLPK_OK)
        return rc;
    CLPK_REQUIRE(a, "args is NULL");
    KindInfo ki;
    CLPK_REQUIRE(kind_info(a->kind, &ki), "unknown kind %d", a->kind);
    CLPK_REQUIRE(a->d_a && a->d_b && a->d_status, "NULL buffer");
    CLPK_REQUIRE(((uintptr_t)a->d_a % 16) == 0 && ((uintptr_t)a->d_b % 16) == 0, "tiles must be 16-byte aligned");
    CLPK_REQUIRE(a->n_mma >= 1 && a->grid >= 1, "n_mma and grid must be >= 1");
    CLPK_REQUIRE(a->n_out_tiles <= a->grid, "n_out_tiles exceeds grid");
    CLPK_REQUIRE(a->n_out_tiles == 0 || (a->d_out && ((uintptr_t)a->d_out % 16) == 0), "d_out missing or misaligned");
    if (ki.scaled)
        CLPK_REQUIRE(a->d_sfa && a->d_sfb, "block-scaled kinds need d_sfa and d_sfb");
    if (ki.sparse) {
        CLPK_REQUIRE(a->d_meta && ((uintptr_t)a->d_meta % 4) == 0, "sparse kinds need d_meta (4-byte aligned)");
    }
    cudaStream_t s = as_stream(stream);
    CLPK_CUDA(cudaMemsetAsync(a->d_status, 0, sizeof(uint32_t), s));
    PeakParams p;
    p.a = static_cast<const uint8_t *>(a->d_a);
    p.b = static_cast<const uint8_t *>(a->d_b);
    p.sfa = static_cast<const uint8_t *>(a->d_sfa);
    p.sfb = static_cast<const uint8_t *>(a->d_sfb);
    p.meta = static_cast<const uint8_t *>(a->d_meta);
    p.n_mma = a->n_mma;
    p.n_out_tiles = a->n_out_tiles;
    p.out = static_cast<uint32_t *>(a->d_out);
    p.checksum = a->d_checksum;
    p.status = a->d_status;
    p.clock = a->d_clock;
    p.lone_lane = tuning(CLPK_TUNE_MMA_LONE_LANE) == 1 ? 1u : 0u;
    switch (a->kind) {
    case CLPK_MMA_E4M3_SP: return launch_peak_sparse<CLPK_MMA_E4M3_SP>(p, a->grid, (uint32_t)ki.k / 32, s);
    case CLPK_MMA_I8_SP:   return launch_peak_sparse<CLPK_MMA_I8_SP>(p, a->grid, (uint32_t)ki.k / 32, s);
    case CLPK_MMA_MXF4_SP: return launch_peak_sparse<CLPK_MMA_MXF4_SP>(p, a->grid, 2, s);
    case CLPK_MMA_NVF4_SP: return launch_peak_sparse<CLPK_MMA_NVF4_SP>(p, a->grid, 2, s);
    case CLPK_MMA_F16:  return launch_peak<CLPK_MMA_F16>(p, a->grid, s);
    case CLPK_MMA_BF16: return launch_peak<CLPK_MMA_BF16>(p, a->grid, s);
    case CLPK_MMA_E4M3: return launch_peak<CLPK_MMA_E4M3>(p, a->grid, s);
    case CLPK_MMA_E5M2: return launch_peak<CLPK_MMA_E5M2>(p, a->grid, s);
    case CLPK_MMA_I8:   return launch_peak<CLPK_MMA_I8>(p, a->grid, s);
    case CLPK_MMA_TF32: return launch_peak<CLPK_MMA_TF32>(p, a->grid, s);
    case CLPK_MMA_F16_F16: return launch_peak<CLPK_MMA_F16_F16>(p, a->grid, s);
    case CLPK_MMA_E2M1: return launch_peak<CLPK_MMA_E2M1>(p, a->grid, s);
    case CLPK_MMA_MXF4: return launch_peak<CLPK_MMA_MXF4>(p, a->grid, s);
    case CLPK_MMA_NVF4: return launch_peak<CLPK_MMA_NVF4>(p, a->grid, s);
    default: break;
    }
    set_error("kind %d not handled", a->kind);
    return CLPK_ERR_BAD_ARG;
}

} // extern "C"
