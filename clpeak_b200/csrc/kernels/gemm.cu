// C[M][N] = A[M][K] * B[N][K]^T on tcgen05.mma, the in-house replacement for the
// cuBLASLt call the reference makes for its "GEMM peak" rows.
//
// Shape of the dense kernel (gemm_kernel; the block-scaled FP4 kernel further down
// keeps a 256 x 256 cluster tile because its scale factors need tensor-memory columns)
//  * Persistent: one 2-CTA cluster per SM pair, tiles handed out round-robin.
//  * A cluster computes a 512 x 256 tile with 2-SM MMAs (cta_group::2, M = 256,
//    N = 256), two row blocks sharing one B tile; each CTA holds 256 x 256 of the
//    accumulator, i.e. all of its tensor memory.  The MMA reads both CTAs' shared
//    memory.  No TMA multicast anywhere: each CTA fetches what it needs itself.
//  * Warp roles (320 threads): warp 0 TMA producer, warp 1 MMA issuer (leader
//    CTA only) and TMEM owner, warps 2-9 epilogue (TMEM -> registers -> output
//    type -> swizzled staging box in shared memory -> TMA store).  The roles
//    that issue TMA or tcgen05 instructions run their loops as whole warps and
//    let one elected lane issue.
//  * K is consumed in blocks of 128 bytes per row (64 x 16-bit, 128 x 8-bit),
//    the width of one 128-byte-swizzled TMA box; a stage is two 16 KiB A
//    sub-tiles (one per row block) and this CTA's 16 KiB half of B, four
//    stages.  Both CTAs' loads signal the leader's "full" barrier;
//    tcgen05.commit releases a stage in both CTAs at once.
//  * Every mbarrier wait is bounded; on expiry the status word is set and all
//    roles fall through to the common exit, which frees tensor memory.
//
// Algorithmic work: 2*M*N*K flop per call; HBM traffic at least
// (M*K + N*K)*elem + M*N*2 bytes (each operand read once, C written once).
#include <cuda.h>
#include <cuda_bf16.h>

#include <atomic>
#include <cstdlib>

#include "../clpk_internal.h"
#include "../clpk_ptx.cuh"

namespace clpk {

constexpr uint32_t kRowBytesK = 128;                        // K bytes per row per stage
constexpr uint32_t kHalfTileBytes = 128 * kRowBytesK;       // 16 KiB: 128 rows x 128 B
constexpr uint32_t kStageBytes = 2 * kHalfTileBytes;        // A half + B half (block-scaled kernel)
constexpr uint32_t kTileMN = 256;
constexpr int kGemmThreads = 320;                          // dense kernel: producer, MMA, 8 epilogue warps

struct GemmParams {
    uint32_t m, n, k;
    uint32_t k_blocks;          // K / (elements per 128 B)
    uint32_t k_block_elems;
    void *c;                    // bf16, or fp32 (TF32) / int32 (I8): see out_elem_bytes()
    float alpha;
    uint32_t *status;
    uint32_t group;             // tile columns per raster group (both kernels)
    unsigned int *wave_sync;    // one counter for this launch, or NULL: see wave_align()
    uint32_t align_at;          // K block of a tile before which the producers meet
    uint32_t align_period;      // ... in every align_period-th wave
    unsigned long long *clock;  // two words: CTA 0 stores the SM cycles and nanoseconds it ran for (clpk_gemm_last_clock)
    uint32_t zero_status;       // 1: the kernel clears *status itself (launches that may overlap the previous kernel's tail)
};

// Launches of a small GEMM repeat every 40-100 us, and 6-7 us of each are the CTA's set-up (barriers, tensor
// memory, descriptor prefetch) and the launch gap.  The plain (non-cooperative) launches therefore carry the
// programmatic-serialisation attribute: a CTA of launch i + 1 takes an SM as soon as launch i's CTA there has
// exited, does its set-up, and then waits here until launch i has completed as a whole and its writes are visible.
// Nothing of global memory is read or written before that point.
__device__ __forceinline__ void join_previous_launch(const GemmParams &p)
{
    griddep_wait();
    if (p.zero_status && blockIdx.x == 0 && threadIdx.x == 0)
        *p.status = 0u;
    griddep_launch_dependents();
}

// Output element of a GEMM dtype: fp32 for TF32, int32 for I8, bf16 for everything else.
template <int DT> struct OutBytes { static constexpr uint32_t value = (DT == CLPK_DT_TF32 || DT == CLPK_DT_I8) ? 4u : 2u; };

// Thread-local epilogue step: 32 consecutive accumulator columns of one row -> global memory.
template <int DT>
__device__ __forceinline__ void store_columns(uint8_t *dst_bytes, const uint32_t (&r)[32], float alpha)
{
    if constexpr (DT == CLPK_DT_I8) {
        uint4 *dst = reinterpret_cast<uint4 *>(dst_bytes);
#pragma unroll
        for (int i = 0; i < 8; i++)
            dst[i] = make_uint4(r[4 * i], r[4 * i + 1], r[4 * i + 2], r[4 * i + 3]);
    } else if constexpr (DT == CLPK_DT_TF32) {
        uint4 *dst = reinterpret_cast<uint4 *>(dst_bytes);
#pragma unroll
        for (int i = 0; i < 8; i++)
            dst[i] = make_uint4(__float_as_uint(__uint_as_float(r[4 * i]) * alpha), __float_as_uint(__uint_as_float(r[4 * i + 1]) * alpha),
                                __float_as_uint(__uint_as_float(r[4 * i + 2]) * alpha), __float_as_uint(__uint_as_float(r[4 * i + 3]) * alpha));
    } else {
        uint32_t w[16];
#pragma unroll
        for (int i = 0; i < 16; i++) {
            __nv_bfloat162 v = __floats2bfloat162_rn(__uint_as_float(r[2 * i]) * alpha, __uint_as_float(r[2 * i + 1]) * alpha);
            w[i] = *reinterpret_cast<uint32_t *>(&v);
        }
        uint4 *dst = reinterpret_cast<uint4 *>(dst_bytes);
#pragma unroll
        for (int i = 0; i < 4; i++)
            dst[i] = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
    }
}

// 2-D tile load whose completion bytes go to the barrier at the same offset in
// the pair's leader CTA (cluster rank 0).
__device__ __forceinline__ void tma_load_pair(void *smem_dst, const CUtensorMap *tmap, int32_t x,
                                              int32_t y, uint64_t *bar)
{
    uint32_t leader_bar;
    asm volatile("mapa.shared::cluster.u32 %0, %1, 0;" : "=r"(leader_bar) : "r"(smem_u32(bar)));
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4}], [%2];" ::"r"(smem_u32(smem_dst)),
        "l"(tmap), "r"(leader_bar), "r"(x), "r"(y)
        : "memory");
}

// The same with the leader's barrier address already mapped (mapa hoisted out of the loop).
__device__ __forceinline__ void tma_load_pair_at(void *smem_dst, const CUtensorMap *tmap, int32_t x, int32_t y,
                                                 uint32_t leader_bar)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4}], [%2];" ::"r"(smem_u32(smem_dst)),
        "l"(tmap), "r"(leader_bar), "r"(x), "r"(y)
        : "memory");
}

__device__ __forceinline__ uint32_t leader_addr(const void *p)
{
    uint32_t a;
    asm volatile("mapa.shared::cluster.u32 %0, %1, 0;" : "=r"(a) : "r"(smem_u32(p)));
    return a;
}

// Roles that issue TMA or tcgen05 instructions run their loops with the whole warp and let
// one elected lane issue.  Addresses and descriptors are then warp-uniform values, which is
// what those instructions take.  With the loop inside `if (lane == 0)` each instruction cost
// its thread 110-130 cycles (measured with clock64 around it: four MMAs 460 cycles, against
// 115 this way), and a thread that must issue four MMAs and a commit per 512 tensor-core
// cycles, or eight and a commit per 1024, was the slowest stage of the pipeline.
// warp_wait: every lane waits; the verdict is made uniform so that the warp stays together.
__device__ __forceinline__ bool warp_wait(uint64_t *bar, uint32_t parity)
{
    return __all_sync(0xffffffffu, mbar_wait(bar, parity) ? 1 : 0) != 0;
}

// DT: BF16 / F16 -> kind::f16 (K = 16 per instruction); E4M3 / E5M2 -> kind::f8f6f4 (K = 32);
// TF32 -> kind::tf32 (K = 8, fp32 out); I8 -> kind::i8 (K = 32, int32 out).  Always 128 bytes of K per stage.
//
// Tile shape.  A cluster computes 512 x 256 of C: two M = 256 row blocks ("halves") that
// share one B tile.  Row block h covers cluster rows [256h, 256h + 256); CTA r of the pair
// owns the r-th 128 of them and keeps that part of the accumulator in tensor-memory
// columns [256h, 256h + 256) -- all 512 columns of each CTA are accumulator.  Per stage a
// CTA loads two 16 KiB A sub-tiles and its 16 KiB half of B (48 KiB; four stages), and the
// leader issues eight 2-CTA instructions (2 halves x 4 K steps).  Against a 256 x 256
// cluster tile this reads a third fewer operand bytes per flop from L2 and DRAM and reads
// B from shared memory once for two row blocks; the price is that the accumulator cannot
// be double-buffered, so the epilogue of a tile (a few microseconds per ~200) is exposed.
// Rows of C beyond M (M a multiple of 256 but not of 512) come out of zero-filled TMA boxes
// and are not stored.
constexpr int kDenseStages = 4;
constexpr uint32_t kDenseStageBytes = 3 * kHalfTileBytes;          // A half 0, A half 1, B half
constexpr uint32_t kDenseTileM = 512;

constexpr int kEpilogueWarps = 8;
constexpr uint32_t kStagingBytes = 32 * 128;                       // 32 rows x 128 bytes of C

struct DenseSmem {
    uint64_t full[kDenseStages];
    uint64_t empty[kDenseStages];
    uint64_t tmem_full;
    uint64_t tmem_empty;
    uint32_t tmem_base;
};

// Tiles are walked in groups of `group` tile columns, M fastest inside a group.
__device__ __forceinline__ void dense_tile_coords(uint32_t tile, uint32_t tiles_m, uint32_t tiles_n, uint32_t group,
                                                  uint32_t &mb, uint32_t &nb)
{
    const uint32_t per_group = group * tiles_m;
    const uint32_t g = tile / per_group;
    const uint32_t within = tile - g * per_group;
    const uint32_t first_n = g * group;
    const uint32_t width = (tiles_n - first_n) < group ? (tiles_n - first_n) : group;
    mb = within / width;
    nb = first_n + within % width;
}

// Epilogue of one warp for one tile of the dense kernel: the warp's 32 rows (TMEM lanes) x 128 columns of each
// of the two row blocks, moved in boxes of 128 bytes per row (64 bf16 or 32 fp32/int32 columns): tcgen05.ld ->
// convert -> the warp's own 4 KiB staging box in shared memory, written in the 128-byte swizzle so that the 32
// lanes (one row each) spread over the banks -> one TMA store per box, which writes whole lines of C and clips
// rows and columns beyond M and N.  (A thread-per-row store straight to global memory costs 32 partial-sector
// transactions per instruction and held the drain of a 256 x 256 CTA tile at 8 us.)  `empty_bar` (in the leader
// CTA) is arrived on as soon as the tile's last tcgen05.ld has landed: the next tile may then overwrite tensor
// memory while the tail of the stores is still in flight.
//   taddr0   : tensor-memory address of this warp's lanes, column 0 of its 128 columns, row block 0
//   row0/col0: C coordinates of the same element
// What a tile's hand-over costs was traced with clock64 stamps on 4 clusters at a fixed 1.84 GHz (K from 1024 to
// 16384: a stage costs its 1024 cycles, a tile a constant on top).  The main loop cannot start the next tile
// before tensor memory is free (both row blocks fill all 512 columns), so everything between the tile's last
// instruction retiring and the arrive on `empty_bar` is exposed once per tile.  In the first version of this
// epilogue that was 5 200 cycles, of which the tcgen05.ld themselves were 700 (a probe reads tensor memory at
// 245 bytes per cycle with eight warps): the rest was two staging boxes stored before row block 1 was read (the
// second box waits until TMA has read the first out of shared memory, 800-1400 cycles behind the operand loads),
// and an mbarrier.arrive.release.cluster that took 1 650 cycles to retire because a release waits for the warp's
// earlier shared-memory and bulk stores.  Now every column is read and converted before anything is stored and
// the arrive is relaxed (the hand-over carries no memory): 2 200 cycles, 8192^3 fp8 3.9 % and NVFP4 5.5 % fewer.

// one staging box out: wait until the previous store has read the box, fill it, hand it to TMA
__device__ __forceinline__ void store_staged_box(const uint32_t (&w)[32], uint8_t *box, const CUtensorMap *tmap_c, uint32_t col,
                                                 uint32_t row, int lane)
{
    uint8_t *my_row = box + lane * 128;
    const uint32_t sw = (uint32_t)(lane & 7);
    if (lane == 0)
        bulk_wait_read<0>();
    __syncwarp();
#pragma unroll
    for (uint32_t j = 0; j < 8; j++)
        *reinterpret_cast<uint4 *>(my_row + ((j ^ sw) << 4)) = make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) {
        tma_store_2d(tmap_c, box, (int32_t)col, (int32_t)row);
        bulk_commit();
    }
}

__device__ __forceinline__ void pack_bf16x64(uint32_t (&w)[32], const uint32_t (&r0)[32], const uint32_t (&r1)[32], float alpha)
{
    // The conversion sits between the reads and the release of tensor memory; alpha = 1 (every dense row of the
    // benchmark) skips the 64 multiplies, which are two thirds of its instructions.  x * 1.0f is x, bit for bit.
    if (alpha == 1.0f) {
#pragma unroll
        for (int i = 0; i < 16; i++) {
            __nv_bfloat162 v0 = __floats2bfloat162_rn(__uint_as_float(r0[2 * i]), __uint_as_float(r0[2 * i + 1]));
            __nv_bfloat162 v1 = __floats2bfloat162_rn(__uint_as_float(r1[2 * i]), __uint_as_float(r1[2 * i + 1]));
            w[i] = *reinterpret_cast<uint32_t *>(&v0);
            w[16 + i] = *reinterpret_cast<uint32_t *>(&v1);
        }
        return;
    }
#pragma unroll
    for (int i = 0; i < 16; i++) {
        __nv_bfloat162 v0 = __floats2bfloat162_rn(__uint_as_float(r0[2 * i]) * alpha, __uint_as_float(r0[2 * i + 1]) * alpha);
        __nv_bfloat162 v1 = __floats2bfloat162_rn(__uint_as_float(r1[2 * i]) * alpha, __uint_as_float(r1[2 * i + 1]) * alpha);
        w[i] = *reinterpret_cast<uint32_t *>(&v0);
        w[16 + i] = *reinterpret_cast<uint32_t *>(&v1);
    }
}

template <int DT>
__device__ __forceinline__ void drain_warp_tile_wide(uint32_t taddr0, uint32_t row0, uint32_t col0, uint8_t *box,
                                                     const CUtensorMap *tmap_c, float alpha, uint64_t *empty_bar, int lane)
{
    // The hand-over carries no memory (the reads have completed: tcgen05.wait::ld), so the arrive needs no release:
    // with it the instruction took 1 650 cycles to retire here -- it waits for the warp's earlier shared-memory and
    // bulk stores -- against 400 without.
    auto release = [&]() {
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0)
            mbar_arrive_cluster_relaxed(empty_bar, 0);
    };
    if constexpr (OutBytes<DT>::value == 2) {
        // 16-bit outputs: every column of the warp's lanes is read and packed (128 registers) before anything is
        // written out, so that tensor memory is held for the reads alone: row block 0 with four tcgen05.ld in
        // flight, row block 1 in two rounds of two (the register file holds no more).
        uint32_t w0[32], w1[32], w2[32], w3[32];
        {
            uint32_t r0[32], r1[32], r2[32], r3[32];
            tmem_ld_32x32b_x32(taddr0, r0);
            tmem_ld_32x32b_x32(taddr0 + 32, r1);
            tmem_ld_32x32b_x32(taddr0 + 64, r2);
            tmem_ld_32x32b_x32(taddr0 + 96, r3);
            tmem_ld_wait();
            pack_bf16x64(w0, r0, r1, alpha);
            pack_bf16x64(w1, r2, r3, alpha);
        }
        {
            uint32_t r0[32], r1[32];
            tmem_ld_32x32b_x32(taddr0 + 256, r0);
            tmem_ld_32x32b_x32(taddr0 + 256 + 32, r1);
            tmem_ld_wait();
            pack_bf16x64(w2, r0, r1, alpha);
        }
        {
            uint32_t r0[32], r1[32];
            tmem_ld_32x32b_x32(taddr0 + 256 + 64, r0);
            tmem_ld_32x32b_x32(taddr0 + 256 + 96, r1);
            tmem_ld_wait();
            release();
            pack_bf16x64(w3, r0, r1, alpha);
        }
        store_staged_box(w0, box, tmap_c, col0, row0, lane);
        store_staged_box(w1, box, tmap_c, col0 + 64, row0, lane);
        store_staged_box(w2, box, tmap_c, col0, row0 + 256, lane);
        store_staged_box(w3, box, tmap_c, col0 + 64, row0 + 256, lane);
    } else {
        // 32-bit outputs: a row block's 128 columns per round, four boxes of 32 columns
#pragma unroll 1
        for (uint32_t h = 0; h < 2; h++) {
            uint32_t r0[32], r1[32], r2[32], r3[32];
            tmem_ld_32x32b_x32(taddr0 + h * 256, r0);
            tmem_ld_32x32b_x32(taddr0 + h * 256 + 32, r1);
            tmem_ld_32x32b_x32(taddr0 + h * 256 + 64, r2);
            tmem_ld_32x32b_x32(taddr0 + h * 256 + 96, r3);
            tmem_ld_wait();
            if (h == 1)
                release();
            if constexpr (DT == CLPK_DT_TF32) {
#pragma unroll
                for (int i = 0; i < 32; i++) {
                    r0[i] = __float_as_uint(__uint_as_float(r0[i]) * alpha);
                    r1[i] = __float_as_uint(__uint_as_float(r1[i]) * alpha);
                    r2[i] = __float_as_uint(__uint_as_float(r2[i]) * alpha);
                    r3[i] = __float_as_uint(__uint_as_float(r3[i]) * alpha);
                }
            }
            store_staged_box(r0, box, tmap_c, col0, row0 + h * 256, lane);
            store_staged_box(r1, box, tmap_c, col0 + 32, row0 + h * 256, lane);
            store_staged_box(r2, box, tmap_c, col0 + 64, row0 + h * 256, lane);
            store_staged_box(r3, box, tmap_c, col0 + 96, row0 + h * 256, lane);
        }
    }
}

// The same for a kernel with a single accumulator (bf16 output, one row block), where the
// next tile's main loop cannot start before tensor memory is free: all 128 columns are read
// and tensor memory is released before anything is written out.  Two rounds of two
// tcgen05.ld (64 fp32 registers in flight, 32 packed ones kept) rather than one of four,
// which would not fit the register file.
// ROUNDS = boxes of 64 columns this warp owns: 2 (a 128-column share) or 1 (a 64-column share).
template <int ROUNDS>
__device__ __forceinline__ void drain_warp_tile_early(uint32_t taddr0, uint32_t row0, uint32_t col0, uint8_t *box,
                                                      const CUtensorMap *tmap_c, float alpha, uint64_t *empty_bar,
                                                      int lane)
{
    uint8_t *my_row = box + lane * 128;
    const uint32_t sw = (uint32_t)(lane & 7);
    uint32_t w[ROUNDS][32];
#pragma unroll
    for (uint32_t b = 0; b < ROUNDS; b++) {
        uint32_t r0[32], r1[32];
        tmem_ld_32x32b_x32(taddr0 + b * 64, r0);
        tmem_ld_32x32b_x32(taddr0 + b * 64 + 32, r1);
        tmem_ld_wait();
        if (b == ROUNDS - 1) {
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0)
                mbar_arrive_cluster_relaxed(empty_bar, 0);      // see drain_warp_tile_wide
        }
#pragma unroll
        for (int i = 0; i < 16; i++) {
            __nv_bfloat162 v0 = __floats2bfloat162_rn(__uint_as_float(r0[2 * i]) * alpha, __uint_as_float(r0[2 * i + 1]) * alpha);
            __nv_bfloat162 v1 = __floats2bfloat162_rn(__uint_as_float(r1[2 * i]) * alpha, __uint_as_float(r1[2 * i + 1]) * alpha);
            w[b][i] = *reinterpret_cast<uint32_t *>(&v0);
            w[b][16 + i] = *reinterpret_cast<uint32_t *>(&v1);
        }
    }
#pragma unroll
    for (uint32_t b = 0; b < ROUNDS; b++) {
        // the previous box must have been read out of shared memory by its store
        if (lane == 0)
            bulk_wait_read<0>();
        __syncwarp();
#pragma unroll
        for (uint32_t j = 0; j < 8; j++)
            *reinterpret_cast<uint4 *>(my_row + ((j ^ sw) << 4)) =
                make_uint4(w[b][4 * j], w[b][4 * j + 1], w[b][4 * j + 2], w[b][4 * j + 3]);
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
            tma_store_2d(tmap_c, box, (int32_t)(col0 + b * 64), (int32_t)row0);
            bulk_commit();
        }
    }
}

// Keeping the clusters in step.  The schedule is static, so all clusters start wave w
// (their w-th tile) together only if they run at exactly the same speed.  They do not:
// measured on a B200, the start times of a wave spread by about 4 us more with every
// wave (some SM pairs are persistently ~1.7 % slower), 70 us after 20 waves.  Clusters
// that share an operand panel then ask for it that far apart, the L2 has long replaced
// it, and every panel is fetched from DRAM several times per wave.  So the producers
// meet before each wave: every CTA adds one to a counter and waits until the counter
// shows that all CTAs of the wave have arrived.  The kernel is launched cooperatively
// (all CTAs resident), and the wait is bounded all the same: a CTA that has waited
// 40 us stops taking part, after which the others time out once each and the kernel
// finishes unaligned.
__device__ __forceinline__ void wave_align(const GemmParams &p, uint32_t wave, uint32_t n_tiles, uint32_t n_clusters,
                                           bool &enabled)
{
    // every align_period-th wave (short tiles drift less per wave and a meeting costs about a microsecond)
    if (!enabled || wave == 0 || wave % p.align_period != 0)
        return;
    // arrivals expected up to and including this meeting: two CTAs per cluster for each earlier
    // meeting (those waves were full) plus two per tile of this wave
    const uint32_t in_wave = n_tiles - wave * n_clusters < n_clusters ? n_tiles - wave * n_clusters : n_clusters;
    const unsigned int target = 2u * (n_clusters * (wave / p.align_period - 1u) + in_wave);
    atomicAdd(p.wave_sync, 1u);
    unsigned long long t0, t1;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    for (;;) {
        unsigned int seen;
        asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(p.wave_sync) : "memory");
        if (seen >= target)
            return;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
        if (t1 - t0 > 40000ull) {
            enabled = false;
            return;
        }
        __nanosleep(64);
    }
}

template <int DT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads)
    gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                const __grid_constant__ CUtensorMap tmap_c, GemmParams p)
{
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    // The runtime only guarantees 16-byte alignment of dynamic shared memory;
    // the swizzled tiles need 1024.
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *staging = smem + (size_t)kDenseStages * kDenseStageBytes;           // one 4 KiB box per epilogue warp
    DenseSmem *sh = reinterpret_cast<DenseSmem *>(staging + kEpilogueWarps * kStagingBytes);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const uint32_t cluster_id = blockIdx.x >> 1;
    const uint32_t n_clusters = gridDim.x >> 1;
    const uint32_t tiles_m = (p.m + kDenseTileM - 1) / kDenseTileM, tiles_n = (p.n + kTileMN - 1) / kTileMN;
    const uint32_t n_tiles = tiles_m * tiles_n;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kDenseStages; s++) {
            mbar_init(&sh->full[s], 1);
            mbar_init(&sh->empty[s], 1);
        }
        mbar_init(&sh->tmem_full, 1);
        mbar_init(&sh->tmem_empty, 16);      // 8 epilogue warps x 2 CTAs
        mbar_fence_init();
        tma_prefetch_desc(&tmap_a);
        tma_prefetch_desc(&tmap_b);
        tma_prefetch_desc(&tmap_c);
    }
    if (warp == 1)
        tmem_alloc<2>(&sh->tmem_base, 512);
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync();
    tc_fence_after_sync();
    const uint32_t tmem = sh->tmem_base;
    join_previous_launch(p);
    const unsigned long long clk0 = clock64(), ns0 = globaltimer_ns();

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        {
            const uint32_t full0 = leader_addr(&sh->full[0]);      // barriers are 8 bytes apart
            uint32_t it = 0;
            bool ok = true, aligned = p.wave_sync != nullptr;
            for (uint32_t tile = cluster_id; tile < n_tiles && ok; tile += n_clusters) {
                uint32_t mb, nb;
                dense_tile_coords(tile, tiles_m, tiles_n, p.group, mb, nb);
                const int32_t row_a0 = (int32_t)(mb * kDenseTileM + rank * 128);
                const int32_t row_b = (int32_t)(nb * kTileMN + rank * 128);
                // Meet the other producers after the tile's first two stages are on their way, not
                // before: the MMA thread then has work while the slowest producer arrives.
                const uint32_t align_at = p.k_blocks > p.align_at ? p.align_at : 0u;
                for (uint32_t kb = 0; kb < p.k_blocks; kb++, it++) {
                    if (kb == align_at) {
                        if (lane == 0)
                            wave_align(p, tile / n_clusters, n_tiles, n_clusters, aligned);
                        aligned = __shfl_sync(0xffffffffu, aligned ? 1 : 0, 0) != 0;
                    }
                    const uint32_t s = it % kDenseStages, round = it / kDenseStages;
                    if (round > 0 && !warp_wait(&sh->empty[s], (round - 1) & 1)) {
                        if (lane == 0)
                            atomicCAS(p.status, 0u, 0x201u);
                        ok = false;
                        break;
                    }
                    uint8_t *st = smem + (size_t)s * kDenseStageBytes;
                    const int32_t x = (int32_t)(kb * p.k_block_elems);
                    if (elect_one()) {
                        if (rank == 0)
                            mbar_expect_tx(&sh->full[s], 2 * kDenseStageBytes);
                        tma_load_pair_at(st, &tmap_a, x, row_a0, full0 + 8 * s);
                        tma_load_pair_at(st + kHalfTileBytes, &tmap_a, x, row_a0 + 256, full0 + 8 * s);
                        tma_load_pair_at(st + 2 * kHalfTileBytes, &tmap_b, x, row_b, full0 + 8 * s);
                    }
                    __syncwarp();
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer (leader CTA) ----------------
        if (rank == 0) {
            constexpr uint32_t kAFmt = DT == CLPK_DT_BF16 ? kFmtBF16 : DT == CLPK_DT_F16 ? kFmtF16 : DT == CLPK_DT_TF32 ? kFmtTF32
                                     : DT == CLPK_DT_I8 ? kFmtS8 : DT == CLPK_DT_E5M2 ? kFmtE5M2 : kFmtE4M3;
            // the E5M2 variant multiplies e5m2 A by e4m3 B (the pairing the reference's fp8_e5m2 row uses)
            constexpr uint32_t kBFmt = DT == CLPK_DT_E5M2 ? kFmtE4M3 : kAFmt;
            const uint32_t idesc = make_idesc(256, 256, kAFmt, kBFmt, DT == CLPK_DT_I8 ? kAccS32 : kAccF32);
            uint32_t it = 0, tcount = 0;
            bool ok = true;
            for (uint32_t tile = cluster_id; tile < n_tiles && ok; tile += n_clusters, tcount++) {
                if (tcount > 0 && !warp_wait(&sh->tmem_empty, (tcount - 1) & 1)) {
                    if (lane == 0)
                        atomicCAS(p.status, 0u, 0x202u);
                    break;
                }
                tc_fence_after_sync();
                for (uint32_t kb = 0; kb < p.k_blocks; kb++, it++) {
                    const uint32_t s = it % kDenseStages, round = it / kDenseStages;
                    if (!warp_wait(&sh->full[s], round & 1)) {
                        if (lane == 0)
                            atomicCAS(p.status, 0u, 0x203u);
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    const uint32_t base = smem_u32(smem + (size_t)s * kDenseStageBytes);
                    const uint64_t bd = make_smem_desc(base + 2 * kHalfTileBytes, 16, 1024, kSwizzle128B);
                    if (elect_one()) {
#pragma unroll
                        for (uint32_t h = 0; h < 2; h++) {
                            const uint64_t ad = make_smem_desc(base + h * kHalfTileBytes, 16, 1024, kSwizzle128B);
                            const uint32_t d = tmem + h * 256;
#pragma unroll
                            for (uint32_t kk = 0; kk < 4; kk++) {
                                // +32 bytes of K per instruction: +2 in the (>>4) address field
                                if constexpr (DT == CLPK_DT_E4M3 || DT == CLPK_DT_E5M2)
                                    mma2_f8f6f4_ss(d, ad + 2 * kk, bd + 2 * kk, idesc, (kb | kk) ? 1u : 0u);
                                else if constexpr (DT == CLPK_DT_TF32)
                                    mma2_tf32_ss(d, ad + 2 * kk, bd + 2 * kk, idesc, (kb | kk) ? 1u : 0u);
                                else if constexpr (DT == CLPK_DT_I8)
                                    mma2_i8_ss(d, ad + 2 * kk, bd + 2 * kk, idesc, (kb | kk) ? 1u : 0u);
                                else
                                    mma2_f16_ss(d, ad + 2 * kk, bd + 2 * kk, idesc, (kb | kk) ? 1u : 0u);
                            }
                        }
                        tc_commit_pair(&sh->empty[s], 3);
                    }
                    __syncwarp();
                }
                if (ok && elect_one())
                    tc_commit_pair(&sh->tmem_full, 3);
                __syncwarp();
            }
        }
    } else {
        // ---------------- epilogue warps ----------------
        // Eight warps: warp w may read TMEM lanes 32 (w % 4) .. +31; the two warps of a lane
        // quarter split each row block's 256 columns in halves (drain_warp_tile).
        const uint32_t q = (uint32_t)(warp & 3);
        const uint32_t col_half = (uint32_t)(warp - 2) >> 2;
        uint8_t *box = staging + (size_t)(warp - 2) * kStagingBytes;
        uint32_t tcount = 0;
        for (uint32_t tile = cluster_id; tile < n_tiles; tile += n_clusters, tcount++) {
            uint32_t mb, nb;
            dense_tile_coords(tile, tiles_m, tiles_n, p.group, mb, nb);
            // warp-uniform verdict: the tcgen05.ld below is warp-aligned
            if (!__all_sync(0xffffffffu, mbar_wait(&sh->tmem_full, tcount & 1) ? 1 : 0)) {
                if (lane == 0)
                    atomicCAS(p.status, 0u, 0x204u);
                break;
            }
            tc_fence_after_sync();
            drain_warp_tile_wide<DT>(tmem + col_half * 128 + ((q * 32) << 16), mb * kDenseTileM + rank * 128 + q * 32,
                                     nb * kTileMN + col_half * 128, box, &tmap_c, p.alpha, &sh->tmem_empty, lane);
        }
        // The staging box must have been read before this CTA's shared memory goes away; the writes themselves
        // complete like any other store before the grid is reported finished, so they are not waited for here
        // (that wait was about a microsecond at the end of every launch).
        if (lane == 0)
            bulk_wait_read<0>();
    }

    tc_fence_before_sync();
    __syncthreads();
    cluster_sync();
    if (blockIdx.x == 0 && threadIdx.x == 0 && p.clock) {
        p.clock[0] = clock64() - clk0;
        p.clock[1] = globaltimer_ns() - ns0;
    }
    if (warp == 1)
        tmem_dealloc<2>(tmem, 512);
}


// ---------------------------------------------------------------------------------
// NVFP4 GEMM: e2m1 operands, one ue4m3 scale per 16 elements along K
// ---------------------------------------------------------------------------------
//
// Same skeleton as gemm_kernel (2-CTA clusters, TMA ring, one MMA thread, eight epilogue
// warps) with these differences:
//  * 256 x 256 tile per cluster, one accumulator.  K per stage is 256 elements (128 bytes
//    of packed fp4) = four tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X
//    (K = 64), 512 tensor-core cycles.
//  * Every stage also carries scale factors: 2 KiB for this CTA's 128 rows of A
//    and 4 KiB for all 256 columns of B (each CTA of the pair needs B's scales for
//    the whole tile), pre-arranged in global memory in the order tensor memory
//    wants them: per instruction a 512-byte block of 32 rows x 16 bytes, byte
//    (r % 32) * 16 + (r / 32) * 4 + j for row r's j-th factor.  One
//    tcgen05.cp.cta_group::2.32x128b.warpx4 per block copies it from shared to
//    tensor memory in both CTAs (4 columns, replicated in the four lane quarters).
//  * Twelve such copies are needed per stage (six for MXFP4).  The MMA warp issues them itself, in front of the
//    stage's four instructions: tcgen05.cp and tcgen05.mma of one thread run in the order they were issued, so no
//    barrier sits between a stage's factors reaching tensor memory and its multiplies.  (Four dedicated copy warps
//    handing over through an mbarrier were the first design: a stage's copies could start only when the ring's
//    previous pass over that stage had retired -- its tensor-memory columns -- and then queued behind the four
//    stages of instructions issued meanwhile, so the pipe ran dry once per ring: 585 cycles per 512-cycle stage.
//    With the copies in line MXFP4 runs at 513 and NVFP4 at 552: a copy takes about 3 cycles of the pipe, and
//    issuing a stage's seventeen instructions takes the elected lane 304 cycles, eleven 234.)  Writing the factors
//    through registers (tcgen05.st from both CTAs) was
//    tried and is slower: the per-stage cross-CTA mbarrier arrive costs about a microsecond.
//  * Two producer warps per CTA: one loads the A and B tiles (full / empty), one the scale factors (sf_full); both
//    reuse a stage when its instructions have retired (empty).
//  * Tensor memory (256-wide tile): accumulator in columns [0,256), then one 48-column scale area
//    per pipeline stage (16 columns A, 32 columns B).  No room is left for a second
//    accumulator, so a tile's epilogue is not overlapped with the next main loop; the
//    epilogue therefore reads all of its columns and releases tensor memory before it
//    writes anything out (drain_warp_tile_early).  The 128-wide tile (TN = 128) has two
//    128-column accumulators and overlaps the epilogue completely.
//  * MXFP4 (MX = true: kind::mxf4.block_scale.scale_vec::2X, one ue8m0 scale per 32
//    elements) has two factors per row per instruction, so one 32-bit word serves
//    two instructions: the instruction descriptor's scale-factor id picks bytes 0-1
//    or 2-3.  Half the blocks (2 of A + 4 of B per stage), half the copies.
//  * What it costs, in CTA 0's own cycles (clock64 and %globaltimer around the whole kernel,
//    clpk_gemm_last_clock) on 4 clusters at a fixed 1.84 GHz with K from 1024 to 16384: a stage 552 cycles
//    (NVFP4; MXFP4 513) against the 512 of its four instructions -- each scale copy takes about 3 cycles of the
//    pipe -- and a tile about 1 600 more for the hand-over of tensor memory (see drain_warp_tile_wide).  The
//    128-wide tile hides the hand-over but reads A twice as often and is 35 % slower; two N = 128 instructions per K
//    step on the 256-wide tile cost 7 %.  Without effect: an L2 prefetch cursor ahead of the loads (slower), parked
//    mbarrier waits, one polling lane per epilogue warp, raster group widths from 4 to 32, four stages instead of
//    five (3 %), C stored with the L2 evict-first policy.

constexpr int kNvMaxStages = 6;
constexpr int kNvGemmThreads = 32 * (3 + kEpilogueWarps);                   // operand producer, MMA, 8 epilogue warps, scale producer
constexpr uint32_t kNvSfCol = 256;                             // first scale column: after the accumulator(s)

// TN = width of the cluster tile in columns of C.
//   TN = 256: 256 x 256 tile, ONE accumulator (256 columns) and five 48-column scale areas.  Every operand
//             byte is used for 256 outputs, the least L2 traffic per flop; the epilogue of a tile is exposed.
//   TN = 128: 256 x 128 tile, TWO accumulators (2 x 128 columns) and six 32-column scale areas, 448 columns
//             in all.  The epilogue of tile t drains one accumulator while the main loop of tile t + 1 fills
//             the other; the price is half again as many operand bytes per flop (A is re-read for every 128
//             columns instead of every 256) and instructions half as long.
template <bool MX, int TN> struct BlockScaled {
    static constexpr uint32_t a_blocks = MX ? 2 : 4;            // 512-byte scale blocks of A per stage (per CTA)
    static constexpr uint32_t b_blocks = (MX ? 4 : 8) * TN / 256; // ... of B (all TN columns)
    static constexpr uint32_t blocks = a_blocks + b_blocks;
    static constexpr uint32_t sf_bytes = blocks * 512;
    static constexpr uint32_t sf_per_kblock = MX ? 8 : 16;      // factors per row per 256 elements of K
    static constexpr uint32_t b_rows = TN / 2;                  // rows of B this CTA stages
    static constexpr uint32_t b_tile_bytes = b_rows * kRowBytesK;
    static constexpr uint32_t tile_bytes = kHalfTileBytes + b_tile_bytes;          // A half + this CTA's part of B
    static constexpr uint32_t stage_bytes = tile_bytes + 2048 + 4096 * TN / 256;   // + room for NVFP4's scale blocks
    static constexpr int stages = TN == 256 ? 5 : 6;
    static constexpr uint32_t n_acc = 256 / TN;                 // accumulators in tensor memory
    static constexpr uint32_t sf_cols = 16 + TN / 8;            // tensor-memory columns per stage: 16 for A, 4 per 128 columns of B per instruction
    static constexpr uint32_t b_cols_per_instr = TN / 32;       // scale columns of B per instruction (NVFP4)
    static constexpr size_t smem_bytes = (size_t)stages * stage_bytes + kEpilogueWarps * kStagingBytes + 512 + 1024;
    static_assert(kNvSfCol + stages * sf_cols <= 512, "tensor memory columns");
    static_assert(stages <= kNvMaxStages, "barrier arrays");
};

struct NvGemmSmem {
    uint64_t full[kNvMaxStages];     // operand tiles of both CTAs landed (leader's barrier)
    uint64_t sf_full[kNvMaxStages];  // scale factors of both CTAs landed (leader's barrier)
    uint64_t empty[kNvMaxStages];    // the stage's MMAs retired (both CTAs)
    uint64_t tmem_full[2];           // per accumulator
    uint64_t tmem_empty[2];
    uint32_t tmem_base;
};
static_assert(sizeof(NvGemmSmem) <= 512, "NvGemmSmem");

// Row-major scale bytes [rows][k / block] -> 512-byte blocks in tensor-memory order, one
// 32-bit word (four factors) per row per block.  NVFP4: 16 factors per row per stage =
// 4 words; MXFP4: 8 factors = 2 words.  words = words per row per stage.
// is_b = 0: blocks ordered [rows/128][k/256][words];  is_b = 1: [rows/256][k/256][words][2].
// One CTA moves 128 rows x 32 words through shared memory: coalesced 128-byte reads along a
// row, coalesced 512-byte writes of whole blocks (a byte-per-thread scatter took 64 us per
// 16 MiB operand, 7 % of a 16384^3 NVFP4 GEMM; this takes a tenth of that).
// Rows at and beyond `rows` (the operand padded up to whole tiles) get zero factors: their elements arrive
// as zeros from the operand's tensor map, and zero times any finite factor is zero.
__global__ void __launch_bounds__(256) pack_scales_kernel(uint32_t *__restrict__ out, const uint32_t *__restrict__ in, uint32_t rows,
                                                          uint32_t words_per_row, uint32_t kblocks, int is_b, uint32_t words)
{
    __shared__ uint32_t tile[128][33];
    const uint32_t row0 = blockIdx.y * 128, w0 = blockIdx.x * 32;
    for (uint32_t i = threadIdx.x; i < 128 * 32; i += 256) {
        const uint32_t r = i >> 5, c = i & 31;
        tile[r][c] = (w0 + c < words_per_row && row0 + r < rows) ? in[(uint64_t)(row0 + r) * words_per_row + w0 + c] : 0u;
    }
    __syncthreads();
    for (uint32_t i = threadIdx.x; i < 32 * 128; i += 256) {
        const uint32_t c = i >> 7, o = i & 127;            // word column of the tile, word of the 512-byte block
        const uint32_t wd = w0 + c;
        if (wd >= words_per_row)
            continue;
        const uint32_t kb = wd / words, kk = wd % words;
        const uint32_t r = (o & 3) * 32 + (o >> 2);         // block byte (r%32)*16 + (r/32)*4 <-> word (r%32)*4 + r/32
        uint64_t block;
        if (!is_b)
            block = ((uint64_t)blockIdx.y * kblocks + kb) * words + kk;
        else
            block = (((uint64_t)(blockIdx.y >> 1) * kblocks + kb) * words + kk) * 2 + (blockIdx.y & 1);
        out[block * 128 + o] = tile[r][c];
    }
}

template <bool MX, int TN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kNvGemmThreads)
    gemm_block_scaled_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                     const __grid_constant__ CUtensorMap tmap_sfa, const __grid_constant__ CUtensorMap tmap_sfb,
                     const __grid_constant__ CUtensorMap tmap_c, GemmParams p)
{
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    using BS = BlockScaled<MX, TN>;
    constexpr int kNvStages = BS::stages;
    constexpr uint32_t kNvStageBytes = BS::stage_bytes, kNvSfColsPerStage = BS::sf_cols;
    uint8_t *staging = smem + (size_t)kNvStages * kNvStageBytes;                 // one 4 KiB box per epilogue warp
    NvGemmSmem *sh = reinterpret_cast<NvGemmSmem *>(staging + kEpilogueWarps * kStagingBytes);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const uint32_t cluster_id = blockIdx.x >> 1;
    const uint32_t n_clusters = gridDim.x >> 1;
    const uint32_t tiles_m = (p.m + kTileMN - 1) / kTileMN, tiles_n = (p.n + TN - 1) / TN;
    const uint32_t n_tiles = tiles_m * tiles_n;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kNvStages; s++) {
            mbar_init(&sh->full[s], 1);
            mbar_init(&sh->sf_full[s], 1);
            mbar_init(&sh->empty[s], 1);
        }
        for (int acc = 0; acc < 2; acc++) {
            mbar_init(&sh->tmem_full[acc], 1);
            mbar_init(&sh->tmem_empty[acc], 2 * kEpilogueWarps);
        }
        mbar_fence_init();
        tma_prefetch_desc(&tmap_a);
        tma_prefetch_desc(&tmap_b);
        tma_prefetch_desc(&tmap_sfa);
        tma_prefetch_desc(&tmap_sfb);
        tma_prefetch_desc(&tmap_c);
    }
    if (warp == 1)
        tmem_alloc<2>(&sh->tmem_base, 512);
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync();
    tc_fence_after_sync();
    const uint32_t tmem = sh->tmem_base;
    join_previous_launch(p);
    const unsigned long long clk0 = clock64(), ns0 = globaltimer_ns();
    constexpr int kScaleProducerWarp = 2 + kEpilogueWarps;

    if (warp == 0) {
        // ---------------- operand producer (both CTAs): A and B tiles ----------------
        // The scale factors have a producer warp of their own (below): their copies on to tensor
        // memory can then start when 6 KiB have landed instead of 70.
        const uint32_t full0 = leader_addr(&sh->full[0]);          // barriers are 8 bytes apart
        uint32_t it = 0;
        bool ok = true, aligned = p.wave_sync != nullptr;
        for (uint32_t tile = cluster_id; tile < n_tiles && ok; tile += n_clusters) {
            uint32_t mb, nb;
            dense_tile_coords(tile, tiles_m, tiles_n, p.group, mb, nb);
            const int32_t row_a = (int32_t)(mb * kTileMN + rank * 128);
            const int32_t row_b = (int32_t)(nb * TN + rank * BS::b_rows);
            const uint32_t align_at = p.k_blocks > p.align_at ? p.align_at : 0u;
            for (uint32_t kb = 0; kb < p.k_blocks; kb++, it++) {
                if (kb == align_at) {
                    if (lane == 0)
                        wave_align(p, tile / n_clusters, n_tiles, n_clusters, aligned);
                    aligned = __shfl_sync(0xffffffffu, aligned ? 1 : 0, 0) != 0;
                }
                const uint32_t s = it % kNvStages, round = it / kNvStages;
                if (round > 0 && !warp_wait(&sh->empty[s], (round - 1) & 1)) {
                    if (lane == 0)
                        atomicCAS(p.status, 0u, 0x211u);
                    ok = false;
                    break;
                }
                uint8_t *st = smem + (size_t)s * kNvStageBytes;
                const int32_t x = (int32_t)(kb * kRowBytesK);
                if (elect_one()) {
                    if (rank == 0)
                        mbar_expect_tx(&sh->full[s], 2 * BS::tile_bytes);
                    tma_load_pair_at(st, &tmap_a, x, row_a, full0 + 8 * s);
                    tma_load_pair_at(st + kHalfTileBytes, &tmap_b, x, row_b, full0 + 8 * s);
                }
                __syncwarp();
            }
        }
    } else if (warp == kScaleProducerWarp) {
        // ---------------- scale-factor producer (both CTAs) ----------------
        // The stage's scale area in shared memory (and its tensor-memory columns) are free again when the previous
        // round's instructions on the stage have retired: the copies run in front of them in the same queue.
        const uint32_t sf_full0 = leader_addr(&sh->sf_full[0]);
        uint32_t it = 0;
        bool ok = true;
        for (uint32_t tile = cluster_id; tile < n_tiles && ok; tile += n_clusters) {
            uint32_t mb, nb;
            dense_tile_coords(tile, tiles_m, tiles_n, p.group, mb, nb);
            const uint32_t sfa_block0 = (mb * 2 + rank) * p.k_blocks * BS::a_blocks;
            const uint32_t sfb_block0 = nb * p.k_blocks * BS::b_blocks;
            for (uint32_t kb = 0; kb < p.k_blocks; kb++, it++) {
                const uint32_t s = it % kNvStages, round = it / kNvStages;
                if (round > 0 && !warp_wait(&sh->empty[s], (round - 1) & 1)) {
                    if (lane == 0)
                        atomicCAS(p.status, 0u, 0x216u);
                    ok = false;
                    break;
                }
                uint8_t *sf = smem + (size_t)s * kNvStageBytes + BS::tile_bytes;
                if (elect_one()) {
                    if (rank == 0)
                        mbar_expect_tx(&sh->sf_full[s], 2 * BS::sf_bytes);
                    tma_load_pair_at(sf, &tmap_sfa, 0, (int32_t)(sfa_block0 + kb * BS::a_blocks), sf_full0 + 8 * s);
                    tma_load_pair_at(sf + BS::a_blocks * 512, &tmap_sfb, 0, (int32_t)(sfb_block0 + kb * BS::b_blocks),
                                     sf_full0 + 8 * s);
                }
                __syncwarp();
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer (leader CTA) ----------------
        // The whole warp runs the loop and waits; one elected lane issues.  Descriptors and
        // addresses are then warp-uniform values, which is what tcgen05 instructions take:
        // with the loop inside `if (lane == 0)` every operand had to be moved over from a
        // per-thread register, and an instruction cost its thread about 110 cycles.
        if (rank == 0) {
            // MXFP4: instruction kk reads bytes 0-1 (id 0) or 2-3 (id 2) of word kk / 2
            const uint32_t idesc = make_idesc_block_scaled(256, TN, kFmtE2M1, kFmtE2M1, MX ? 1u : 0u, 0, 0);
            const uint32_t idesc_hi = make_idesc_block_scaled(256, TN, kFmtE2M1, kFmtE2M1, 1u, 2, 2);
            uint32_t it = 0, tcount = 0;
            bool ok = true;
            for (uint32_t tile = cluster_id; tile < n_tiles && ok; tile += n_clusters, tcount++) {
                // accumulator `acc` is free again when the epilogue of its previous tile has read it out
                const uint32_t acc = tcount % BS::n_acc, use = tcount / BS::n_acc;
                if (use > 0 && !__all_sync(0xffffffffu, mbar_wait(&sh->tmem_empty[acc], (use - 1) & 1) ? 1 : 0)) {
                    if (lane == 0)
                        atomicCAS(p.status, 0u, 0x212u);
                    break;
                }
                tc_fence_after_sync();
                const uint32_t d_t = tmem + acc * TN;
                for (uint32_t kb = 0; kb < p.k_blocks; kb++, it++) {
                    const uint32_t s = it % kNvStages, round = it / kNvStages;
                    // the scale factors usually arrive first (6 KiB against 64): wait for them, then the tiles
                    const bool landed = mbar_wait(&sh->sf_full[s], round & 1) && mbar_wait(&sh->full[s], round & 1);
                    if (!__all_sync(0xffffffffu, landed ? 1 : 0)) {
                        if (lane == 0)
                            atomicCAS(p.status, 0u, 0x213u);
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    const uint32_t base = smem_u32(smem + (size_t)s * kNvStageBytes);
                    const uint32_t sfa_t = tmem + kNvSfCol + s * kNvSfColsPerStage, sfb_t = sfa_t + 16;
                    const uint64_t ad = make_smem_desc(base, 16, 1024, kSwizzle128B);
                    const uint64_t bd = make_smem_desc(base + kHalfTileBytes, 16, 1024, kSwizzle128B);
                    if (elect_one()) {
                        // the stage's scale factors go to tensor memory in front of its instructions, in the same queue:
                        // 512-byte blocks, A's (4 columns each, from column 0), then B's (from column 16)
                        const uint32_t sf_s = base + BS::tile_bytes;
#pragma unroll
                        for (uint32_t blk = 0; blk < BS::blocks; blk++) {
                            const uint32_t col = blk < BS::a_blocks ? 4 * blk : 16 + 4 * (blk - BS::a_blocks);
                            tmem_cp_32x128b_warpx4<2>(sfa_t + col, make_smem_desc(sf_s + blk * 512, 16, 128, kSwizzleNone));
                        }
#pragma unroll
                        for (uint32_t kk = 0; kk < 4; kk++) {
                            if constexpr (MX)
                                mma2_mxf4_bs(d_t, ad + 2 * kk, bd + 2 * kk, (kk & 1) ? idesc_hi : idesc, sfa_t + 4 * (kk / 2),
                                             sfb_t + BS::b_cols_per_instr * (kk / 2), (kb | kk) ? 1u : 0u);
                            else
                                mma2_nvf4_bs(d_t, ad + 2 * kk, bd + 2 * kk, idesc, sfa_t + 4 * kk, sfb_t + BS::b_cols_per_instr * kk,
                                             (kb | kk) ? 1u : 0u);
                        }
                        tc_commit_pair(&sh->empty[s], 3);
                    }
                    __syncwarp();
                }
                if (ok && elect_one())
                    tc_commit_pair(&sh->tmem_full[acc], 3);
                __syncwarp();
            }
        }
    } else {
        // ---------------- epilogue warps: one row block, tensor memory released before the stores ----------------
        const uint32_t q = (uint32_t)(warp & 3);
        const uint32_t col_half = (uint32_t)(warp - 2) >> 2;
        uint8_t *box = staging + (size_t)(warp - 2) * kStagingBytes;
        uint32_t tcount = 0;
        for (uint32_t tile = cluster_id; tile < n_tiles; tile += n_clusters, tcount++) {
            uint32_t mb, nb;
            dense_tile_coords(tile, tiles_m, tiles_n, p.group, mb, nb);
            const uint32_t acc = tcount % BS::n_acc, use = tcount / BS::n_acc;
            if (!__all_sync(0xffffffffu, mbar_wait(&sh->tmem_full[acc], use & 1) ? 1 : 0)) {
                if (lane == 0)
                    atomicCAS(p.status, 0u, 0x214u);
                break;
            }
            tc_fence_after_sync();
            drain_warp_tile_early<TN / 128>(tmem + acc * TN + col_half * (TN / 2) + ((q * 32) << 16), mb * kTileMN + rank * 128 + q * 32,
                                            nb * TN + col_half * (TN / 2), box, &tmap_c, p.alpha, &sh->tmem_empty[acc], lane);
        }
        // The staging box must have been read before this CTA's shared memory goes away; the writes themselves
        // complete like any other store before the grid is reported finished, so they are not waited for here
        // (that wait was about a microsecond at the end of every launch).
        if (lane == 0)
            bulk_wait_read<0>();
    }

    tc_fence_before_sync();
    __syncthreads();
    cluster_sync();
    if (blockIdx.x == 0 && threadIdx.x == 0 && p.clock) {
        p.clock[0] = clock64() - clk0;
        p.clock[1] = globaltimer_ns() - ns0;
    }
    if (warp == 1)
        tmem_dealloc<2>(tmem, 512);
}

// ---- host side -----------------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

static int get_encode_fn(EncodeTiledFn *out)
{
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void *sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        CLPK_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres));
        if (qres != cudaDriverEntryPointSuccess || !sym) {
            set_error("cuTensorMapEncodeTiled is not available from this driver");
            return CLPK_ERR_CUDA;
        }
        fn = reinterpret_cast<EncodeTiledFn>(sym);
    }
    *out = fn;
    return CLPK_OK;
}

// Row-major [rows][row_bytes] operand, box = box_rows (128 unless said otherwise) x 128 bytes, 128-byte swizzle.
static int make_operand_map(CUtensorMap *map, const void *base, uint64_t rows, uint64_t row_bytes, uint32_t box_rows = 128)
{
    EncodeTiledFn enc;
    int rc = get_encode_fn(&enc);
    if (rc != CLPK_OK)
        return rc;
    const cuuint64_t dims[2] = {row_bytes, rows};
    const cuuint64_t strides[1] = {row_bytes};
    const cuuint32_t box[2] = {kRowBytesK, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_error("cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
        return CLPK_ERR_CUDA;
    }
    return CLPK_OK;
}


// C [m][n] row-major for the epilogue's stores: box = 32 rows x 128 bytes, 128-byte swizzle.
static int make_output_map(CUtensorMap *map, void *base, uint64_t m, uint64_t n, int dtype)
{
    EncodeTiledFn enc;
    int rc = get_encode_fn(&enc);
    if (rc != CLPK_OK)
        return rc;
    const bool wide = dtype == CLPK_DT_TF32 || dtype == CLPK_DT_I8;
    const CUtensorMapDataType type = dtype == CLPK_DT_TF32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                   : dtype == CLPK_DT_I8 ? CU_TENSOR_MAP_DATA_TYPE_INT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    const uint32_t elem = wide ? 4 : 2;
    const cuuint64_t dims[2] = {n, m};
    const cuuint64_t strides[1] = {n * elem};
    const cuuint32_t box[2] = {128 / elem, 32};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, type, 2, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_error("cuTensorMapEncodeTiled (output) failed with CUresult %d", (int)r);
        return CLPK_ERR_CUDA;
    }
    return CLPK_OK;
}

// Packed scale factors: rows of 512 bytes (128 x u32); a box is `rows_per_box` consecutive rows.
static int make_scale_map(CUtensorMap *map, const void *base, uint64_t n_rows, uint32_t rows_per_box)
{
    EncodeTiledFn enc;
    int rc = get_encode_fn(&enc);
    if (rc != CLPK_OK)
        return rc;
    const cuuint64_t dims[2] = {128, n_rows};
    const cuuint64_t strides[1] = {512};
    const cuuint32_t box[2] = {128, rows_per_box};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void *>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_error("cuTensorMapEncodeTiled (scales) failed with CUresult %d", (int)r);
        return CLPK_ERR_CUDA;
    }
    return CLPK_OK;
}


constexpr size_t kGemmSmemBytes = (size_t)kDenseStages * kDenseStageBytes + kEpilogueWarps * kStagingBytes + sizeof(DenseSmem) + 1024;

// One wave counter per launch, from a ring of 32 per device so that launches on different streams
// do not share one; zeroed in stream order before the kernel.  The slot index comes from one
// process-wide counter, so a slot is handed out again 32 launches later: with more than 32 aligned
// GEMMs in flight at once on one device (across streams) two running kernels would share a counter.
// That costs alignment, not correctness -- a producer that does not see its wave complete within
// 40 us stops taking part -- but callers that want the alignment keep at most 32 in flight.
constexpr int kSyncSlots = 32;
__device__ unsigned int g_wave_sync[kSyncSlots];
static std::atomic<unsigned> g_next_sync_slot{0};
static thread_local int g_last_aligned = -1;
// {SM cycles, nanoseconds} CTA 0 of the last GEMM launch on this device ran for (both tensor kernels write it).
__device__ unsigned long long g_gemm_clock[2];

// Launches a persistent cluster kernel whose last parameter is GemmParams: cooperatively with a
// fresh wave counter when the alignment is on, plainly (and unaligned) otherwise.
template <typename Kernel, typename... Maps>
static int launch_persistent(Kernel kernel, const char *what, int threads, size_t smem, cudaStream_t s, GemmParams p,
                             uint32_t n_tiles, const Maps &...maps)
{
    CLPK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const int grid = (num_sms() / 2) * 2;
    p.wave_sync = nullptr;
    p.zero_status = 0;
    g_last_aligned = 0;
    CLPK_CUDA(cudaGetSymbolAddress(reinterpret_cast<void **>(&p.clock), g_gemm_clock));
    // nothing to keep in step in the first two waves: small problems skip the counter and its memset
    const bool worth_aligning = n_tiles > 2u * (uint32_t)(grid / 2) * p.align_period;
    if (worth_aligning && tuning(CLPK_TUNE_GEMM_NO_ALIGN) != 1) {
        unsigned int *base = nullptr;
        CLPK_CUDA(cudaGetSymbolAddress(reinterpret_cast<void **>(&base), g_wave_sync));
        p.wave_sync = base + g_next_sync_slot.fetch_add(1) % kSyncSlots;
        CLPK_CUDA(cudaMemsetAsync(p.wave_sync, 0, sizeof(unsigned int), s));
        CLPK_CUDA(cudaMemsetAsync(p.status, 0, sizeof(uint32_t), s));
        // cooperative: every CTA is resident before any runs, so the wave counter can fill up
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)grid);
        cfg.blockDim = dim3((unsigned)threads);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = s;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeCooperative;
        attr[0].val.cooperative = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        const cudaError_t ce = cudaLaunchKernelEx(&cfg, kernel, maps..., p);
        if (ce == cudaSuccess) {
            g_last_aligned = 1;
            return CLPK_OK;
        }
        // Only "the grid cannot be co-resident here" (another context holds SMs, MPS limits) is a
        // reason to run without the alignment; anything else is a real error and is reported as one.
        if (ce != cudaErrorCooperativeLaunchTooLarge && ce != cudaErrorLaunchOutOfResources)
            return cuda_fail(ce, what);
        (void)cudaGetLastError();
        p.wave_sync = nullptr;
    }
    // No stream operation between two such launches (the kernel clears the status word itself), so that the
    // programmatic serialisation can overlap this launch's set-up with the tail of the one before.
    p.zero_status = 1;
    cudaLaunchConfig_t plain = {};
    plain.gridDim = dim3((unsigned)grid);
    plain.blockDim = dim3((unsigned)threads);
    plain.dynamicSmemBytes = smem;
    plain.stream = s;
    cudaLaunchAttribute pdl[1];
    pdl[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    pdl[0].val.programmaticStreamSerializationAllowed = tuning(CLPK_TUNE_GEMM_NO_PDL) == 1 ? 0 : 1;
    plain.attrs = pdl;
    plain.numAttrs = 1;
    const cudaError_t e = cudaLaunchKernelEx(&plain, kernel, maps..., p);
    if (e != cudaSuccess)
        return cuda_fail(e, what);
    return CLPK_OK;
}

template <int DT>
static int launch_gemm(const CUtensorMap &ta, const CUtensorMap &tb, const CUtensorMap &tc, const GemmParams &p, cudaStream_t s)
{
    const uint32_t n_tiles = ((p.m + kDenseTileM - 1) / kDenseTileM) * ((p.n + kTileMN - 1) / kTileMN);
    return launch_persistent(gemm_kernel<DT>, "gemm", kGemmThreads, kGemmSmemBytes, s, p, n_tiles, ta, tb, tc);
}

} // namespace clpk

using namespace clpk;

extern "C" {

int clpk_gemm_last_launch_aligned(void) { return g_last_aligned; }

int clpk_gemm_last_clock(unsigned long long *h_cycles, unsigned long long *h_ns, void *stream)
{
    CLPK_REQUIRE(h_cycles && h_ns, "NULL output");
    unsigned long long v[2] = {0, 0};
    void *sym = nullptr;
    CLPK_CUDA(cudaGetSymbolAddress(&sym, g_gemm_clock));
    CLPK_CUDA(cudaMemcpyAsync(v, sym, sizeof v, cudaMemcpyDeviceToHost, as_stream(stream)));
    CLPK_CUDA(cudaStreamSynchronize(as_stream(stream)));
    *h_cycles = v[0];
    *h_ns = v[1];
    return CLPK_OK;
}

// rows of a block-scaled operand rounded up to whole 256-row tiles
static inline uint32_t padded_rows(uint32_t rows) { return (rows + 255u) / 256u * 256u; }

int clpk_gemm_workspace_bytes(int dtype, uint32_t m, uint32_t n, uint32_t k, size_t *bytes)
{
    CLPK_REQUIRE(bytes, "bytes is NULL");
    *bytes = 0;
    const size_t rows = (size_t)padded_rows(m) + padded_rows(n);      // scale blocks cover whole tiles
    if (dtype == CLPK_DT_NVF4)
        *bytes = rows * (k / 16);
    if (dtype == CLPK_DT_MXF4)              // packed into 4-byte words of which each instruction uses two bytes
        *bytes = rows * (k / 32);
    return CLPK_OK;
}

// Width of the block-scaled kernel's cluster tile for a problem: 256 (one accumulator, least operand
// traffic) or 128 (two accumulators, the epilogue overlaps the next tile).  The GEMM_FP4_TILE knob
// forces one; the choice also fixes the order of B's scale blocks in the workspace, so a workspace
// packed by clpk_gemm_pack_scales belongs to the knob setting it was packed under.
static uint32_t fp4_tile_n(uint32_t m, uint32_t n, uint32_t k)
{
    const int t = tuning(CLPK_TUNE_GEMM_FP4_TILE);
    if (t == 1)
        return 256;
    if (t == 2)
        return 128;
    (void)m; (void)n; (void)k;
    return 256;
}

// Row-major scale bytes of both operands -> tile order in the workspace (A's blocks, then B's).
static int pack_scales(const clpk_gemm_args_t *a, cudaStream_t s)
{
    const uint32_t words = a->dtype == CLPK_DT_MXF4 ? 2 : 4;   // 32-bit scale words per row per 256 elements of K
    const size_t sfa_bytes = (size_t)padded_rows(a->m) * (a->k / 256) * words * 4, sfb_bytes = (size_t)padded_rows(a->n) * (a->k / 256) * words * 4;
    CLPK_REQUIRE(a->d_sfa && a->d_sfb, "block-scaled FP4 needs d_sfa and d_sfb");
    CLPK_REQUIRE(a->d_workspace && a->workspace_bytes >= sfa_bytes + sfb_bytes && ((uintptr_t)a->d_workspace % 16) == 0,
                 "block-scaled FP4 needs a 16-byte aligned workspace of clpk_gemm_workspace_bytes() bytes");
    CLPK_REQUIRE(((uintptr_t)a->d_sfa % 4) == 0 && ((uintptr_t)a->d_sfb % 4) == 0, "scale arrays must be 4-byte aligned");
    uint8_t *wsa = static_cast<uint8_t *>(a->d_workspace), *wsb = wsa + sfa_bytes;
    const uint32_t words_per_row = a->k / 256 * words, kblocks = a->k / 256;
    const dim3 ga((words_per_row + 31) / 32, padded_rows(a->m) / 128), gb((words_per_row + 31) / 32, padded_rows(a->n) / 128);
    pack_scales_kernel<<<ga, 256, 0, s>>>(reinterpret_cast<uint32_t *>(wsa), static_cast<const uint32_t *>(a->d_sfa), a->m,
                                          words_per_row, kblocks, 0, words);
    // B's blocks: per 256 columns [k block][instruction][column half] for the 256-wide tile, per 128 columns
    // [k block][instruction] (A's order) for the 128-wide one
    pack_scales_kernel<<<gb, 256, 0, s>>>(reinterpret_cast<uint32_t *>(wsb), static_cast<const uint32_t *>(a->d_sfb), a->n,
                                          words_per_row, kblocks, fp4_tile_n(a->m, a->n, a->k) == 256 ? 1 : 0, words);
    CLPK_LAUNCH_CHECK("pack_scales");
    return CLPK_OK;
}

int clpk_gemm_pack_scales(const clpk_gemm_args_t *a, void *stream)
{
    int rc = require_sm100();
    if (rc != CLPK_OK)
        return rc;
    CLPK_REQUIRE(a, "args is NULL");
    CLPK_REQUIRE(a->dtype == CLPK_DT_NVF4 || a->dtype == CLPK_DT_MXF4, "only the block-scaled FP4 kinds have scales to pack");
    CLPK_REQUIRE(a->m > 0 && a->n > 0 && a->k > 0 && a->k % 256 == 0, "M, N positive and K a positive multiple of 256 (got %u, %u, %u)",
                 a->m, a->n, a->k);
    return pack_scales(a, as_stream(stream));
}

int clpk_gemm(const clpk_gemm_args_t *a, void *stream)
{
    int rc = require_sm100();
    if (rc != CLPK_OK)
        return rc;
    CLPK_REQUIRE(a, "args is NULL");
    CLPK_REQUIRE(a->d_a && a->d_b && a->d_c && a->d_status, "NULL buffer");
    if (a->dtype == CLPK_DT_F32 || a->dtype == CLPK_DT_F64) {
        // no tcgen05 kind for these: the CUDA-core fp32 and DMMA fp64 kernels of simt_gemm.cu
        CLPK_CUDA(cudaMemsetAsync(a->d_status, 0, sizeof(uint32_t), as_stream(stream)));
        g_last_aligned = 0;
        return launch_simt_gemm(a->dtype, a->d_a, a->d_b, a->d_c, a->m, a->n, a->k, a->alpha, as_stream(stream));
    }
    CLPK_REQUIRE(a->m > 0 && a->n > 0 && a->k > 0, "M, N and K must be positive");
    const bool block_scaled = a->dtype == CLPK_DT_NVF4 || a->dtype == CLPK_DT_MXF4;
    // Ragged shapes: TMA fills what a box reads beyond the operands with zeros and clips what a box would store
    // beyond C, so a partial tile costs a whole one but needs no code.  The block-scaled kinds keep K in whole
    // stages of 256 elements (four instructions' scale factors travel as one block); their scale blocks are
    // packed for whole tiles, with zero factors for the rows beyond M and N.
    CLPK_REQUIRE(!block_scaled || a->k % 256 == 0, "block-scaled FP4 needs K to be a multiple of 256 (got %u)", a->k);
    CLPK_REQUIRE(((uintptr_t)a->d_a % 16) == 0 && ((uintptr_t)a->d_b % 16) == 0 && ((uintptr_t)a->d_c % 16) == 0,
                 "operands must be 16-byte aligned");
    uint32_t elem_bits;
    switch (a->dtype) {
    case CLPK_DT_BF16:
    case CLPK_DT_F16:  elem_bits = 16; break;
    case CLPK_DT_TF32: elem_bits = 32; break;
    case CLPK_DT_E4M3:
    case CLPK_DT_E5M2:
    case CLPK_DT_I8:   elem_bits = 8; break;
    case CLPK_DT_MXF4:
    case CLPK_DT_NVF4: elem_bits = 4; break;
    default:
        set_error("clpk_gemm: dtype %d is not available in this build", a->dtype);
        return CLPK_ERR_UNSUPPORTED;
    }
    cudaStream_t s = as_stream(stream);

    const uint64_t row_bytes = (uint64_t)a->k * elem_bits / 8;
    CLPK_REQUIRE(((uint64_t)a->k * elem_bits) % (8 * 16) == 0,
                 "K = %u: a row of %u-bit elements must be a multiple of 16 bytes (the pitch of a TMA tensor map)", a->k, elem_bits);
    const uint32_t out_bytes = (a->dtype == CLPK_DT_TF32 || a->dtype == CLPK_DT_I8) ? 4u : 2u;
    CLPK_REQUIRE(((uint64_t)a->n * out_bytes) % 16 == 0, "N = %u: a row of C must be a multiple of 16 bytes", a->n);
    CUtensorMap ta, tb;
    rc = make_operand_map(&ta, a->d_a, a->m, row_bytes);
    if (rc != CLPK_OK)
        return rc;
    rc = make_operand_map(&tb, a->d_b, a->n, row_bytes);
    if (rc != CLPK_OK)
        return rc;

    GemmParams p;
    p.m = a->m;
    p.n = a->n;
    p.k = a->k;
    p.k_block_elems = kRowBytesK;          // x coordinate is in bytes: the maps are typed UINT8
    p.k_blocks = (uint32_t)((row_bytes + kRowBytesK - 1) / kRowBytesK);
    p.c = a->d_c;
    p.alpha = a->alpha;
    p.status = a->d_status;
    // waves of ~(SM pairs) tiles that are about square in elements: twice as many 256-wide tile columns
    // as 512-tall tile rows (74 pairs: 12 x 6)
    p.group = block_scaled ? 8 : 12;          // block-scaled: 256 x 256 tiles, a wave of 74 is about 8 x 9
    p.wave_sync = nullptr;
    p.align_at = 2;
    p.align_period = block_scaled ? 8 : 1;
    if (const int t = tuning(CLPK_TUNE_GEMM_ALIGN_AT); t >= 0)
        p.align_at = (uint32_t)t;
    if (const int t = tuning(CLPK_TUNE_GEMM_GROUP); t > 0)
        p.group = (uint32_t)t;


    if (block_scaled) {
        const bool mx = a->dtype == CLPK_DT_MXF4;
        const uint32_t words = mx ? 2 : 4;                      // 32-bit scale words per row per 256 elements of K
        const size_t sfa_bytes = (size_t)padded_rows(a->m) * (a->k / 256) * words * 4, sfb_bytes = (size_t)padded_rows(a->n) * (a->k / 256) * words * 4;
        CLPK_REQUIRE((a->d_sfa != nullptr) == (a->d_sfb != nullptr), "d_sfa and d_sfb: give both, or neither when the workspace is already packed");
        CLPK_REQUIRE(a->d_workspace && a->workspace_bytes >= sfa_bytes + sfb_bytes && ((uintptr_t)a->d_workspace % 16) == 0,
                     "block-scaled FP4 needs a 16-byte aligned workspace of clpk_gemm_workspace_bytes() bytes");
        uint8_t *wsa = static_cast<uint8_t *>(a->d_workspace), *wsb = wsa + sfa_bytes;
        if (a->d_sfa) {
            rc = pack_scales(a, s);
            if (rc != CLPK_OK)
                return rc;
        }
        const uint32_t tn = fp4_tile_n(a->m, a->n, a->k);
        CUtensorMap tsa, tsb;
        rc = make_scale_map(&tsa, wsa, sfa_bytes / 512, words);
        if (rc != CLPK_OK)
            return rc;
        rc = make_scale_map(&tsb, wsb, sfb_bytes / 512, words * tn / 128);
        if (rc != CLPK_OK)
            return rc;
        CUtensorMap tc;
        rc = make_output_map(&tc, a->d_c, a->m, a->n, a->dtype);
        if (rc != CLPK_OK)
            return rc;
        const uint32_t n_tiles = ((a->m + kTileMN - 1) / kTileMN) * ((a->n + tn - 1) / tn);
        if (tn == 128) {
            rc = make_operand_map(&tb, a->d_b, a->n, row_bytes, 64);       // each CTA stages 64 rows of B per stage
            if (rc != CLPK_OK)
                return rc;
            if (tuning(CLPK_TUNE_GEMM_GROUP) <= 0)
                p.group *= 2;                                              // the same panel width in elements
            p.align_period *= 2;
            return mx ? launch_persistent(gemm_block_scaled_kernel<true, 128>, "gemm_mxf4 (256x128)", kNvGemmThreads,
                                          BlockScaled<true, 128>::smem_bytes, s, p, n_tiles, ta, tb, tsa, tsb, tc)
                      : launch_persistent(gemm_block_scaled_kernel<false, 128>, "gemm_nvf4 (256x128)", kNvGemmThreads,
                                          BlockScaled<false, 128>::smem_bytes, s, p, n_tiles, ta, tb, tsa, tsb, tc);
        }
        return mx ? launch_persistent(gemm_block_scaled_kernel<true, 256>, "gemm_mxf4", kNvGemmThreads,
                                      BlockScaled<true, 256>::smem_bytes, s, p, n_tiles, ta, tb, tsa, tsb, tc)
                  : launch_persistent(gemm_block_scaled_kernel<false, 256>, "gemm_nvf4", kNvGemmThreads,
                                      BlockScaled<false, 256>::smem_bytes, s, p, n_tiles, ta, tb, tsa, tsb, tc);
    }
    CUtensorMap tc;
    rc = make_output_map(&tc, a->d_c, a->m, a->n, a->dtype);
    if (rc != CLPK_OK)
        return rc;
    switch (a->dtype) {
    case CLPK_DT_BF16: return launch_gemm<CLPK_DT_BF16>(ta, tb, tc, p, s);
    case CLPK_DT_F16:  return launch_gemm<CLPK_DT_F16>(ta, tb, tc, p, s);
    case CLPK_DT_TF32: return launch_gemm<CLPK_DT_TF32>(ta, tb, tc, p, s);
    case CLPK_DT_I8:   return launch_gemm<CLPK_DT_I8>(ta, tb, tc, p, s);
    case CLPK_DT_E5M2: return launch_gemm<CLPK_DT_E5M2>(ta, tb, tc, p, s);
    default:           return launch_gemm<CLPK_DT_E4M3>(ta, tb, tc, p, s);
    }
}

} // extern "C"
