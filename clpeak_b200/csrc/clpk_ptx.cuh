// Inline-PTX wrappers for the sm_100a features the kernels use: mbarrier,
// 1-D and tiled bulk copies (TMA), tensor memory (TMEM) management and the
// tcgen05 family.  Only what the kernels in this directory need.
//
// Every wait is bounded: mbar_wait() gives up after a wall-clock budget read
// from %globaltimer and reports failure, so a wrong descriptor or a missing
// arrive turns into an error status instead of a hung GPU.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace clpk {

__device__ __forceinline__ uint32_t smem_u32(const void *p)
{
    return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ uint64_t globaltimer_ns()
{
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ uint32_t elect_one()
{
    uint32_t pred = 0;
    asm volatile(
        "{\n\t"
        ".reg .pred P;\n\t"
        "elect.sync _|P, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, P;\n\t"
        "}\n"
        : "=r"(pred));
    return pred;
}

// ---- programmatic dependent launch -----------------------------------------------
// A kernel launched with cudaLaunchAttributeProgrammaticStreamSerialization may start while the kernel before it
// in the stream is still running.  griddep_wait() blocks until that kernel has completed and its memory
// operations are visible (a no-op in a kernel launched without the attribute); griddep_launch_dependents() lets
// the kernel after this one begin to launch as soon as this one's CTAs make room.

__device__ __forceinline__ void griddep_wait()
{
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

__device__ __forceinline__ void griddep_launch_dependents()
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// ---- mbarrier ---------------------------------------------------------------

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void mbar_fence_init()
{
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
                 "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t *bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// Arrive on the barrier at the same shared-memory offset in CTA `cta` of the cluster, without release semantics:
// for hand-overs that carry no memory (a tensor-memory accumulator whose reads have completed: tcgen05.wait::ld and
// tcgen05.fence::before_thread_sync order those).  A releasing arrive waits for the warp's earlier shared-memory
// and bulk stores and took 1 650 cycles to retire in the GEMM epilogue, this one 400.
__device__ __forceinline__ void mbar_arrive_cluster_relaxed(uint64_t *bar, uint32_t cta)
{
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(bar)), "r"(cta));
    asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(remote) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred P;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, P;\n\t"
        "}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Wall-clock budget for any single device-side wait.
constexpr uint64_t kWaitBudgetNs = 4000000000ull;

// Returns false when the phase did not complete within the budget.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity,
                                          uint64_t budget_ns = kWaitBudgetNs)
{
    if (mbar_try_wait(bar, parity))
        return true;
    const uint64_t t0 = globaltimer_ns();
    uint32_t spins = 0;
    while (true) {
        if (mbar_try_wait(bar, parity))
            return true;
        if ((++spins & 0x3ff) == 0 && globaltimer_ns() - t0 > budget_ns)
            return false;
    }
}

// ---- fences ---------------------------------------------------------------------

// Make generic-proxy writes to shared memory visible to the async proxy
// (TMA, tcgen05.mma operand reads).
__device__ __forceinline__ void fence_proxy_async_smem()
{
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void tc_fence_before_sync()
{
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tc_fence_after_sync()
{
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ---- 1-D bulk copies (no tensor map) ---------------------------------------------

__device__ __forceinline__ void bulk_g2s(void *smem_dst, const void *gmem_src, uint32_t bytes,
                                         uint64_t *bar)
{
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(smem_u32(smem_dst)), "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}

__device__ __forceinline__ void bulk_s2g(void *gmem_dst, const void *smem_src, uint32_t bytes)
{
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gmem_dst),
                 "r"(smem_u32(smem_src)), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ void bulk_commit()
{
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}

template <int N>
__device__ __forceinline__ void bulk_wait_read()
{
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}

template <int N>
__device__ __forceinline__ void bulk_wait()
{
    asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// ---- tiled TMA (tensor map) -------------------------------------------------------

__device__ __forceinline__ void tma_prefetch_desc(const void *tmap)
{
    asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}

__device__ __forceinline__ void tma_store_2d(const void *tmap, const void *smem_src, int32_t x,
                                             int32_t y)
{
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                     tmap),
                 "r"(smem_u32(smem_src)), "r"(x), "r"(y)
                 : "memory");
}

// ---- cluster ----------------------------------------------------------------------

__device__ __forceinline__ uint32_t cluster_ctarank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}

__device__ __forceinline__ void cluster_arrive()
{
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}

__device__ __forceinline__ void cluster_wait()
{
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

__device__ __forceinline__ void cluster_sync()
{
    cluster_arrive();
    cluster_wait();
}

// ---- tensor memory ------------------------------------------------------------------

// One full warp allocates `ncols` (power of two, 32..512) TMEM columns; the base
// address is written to *smem_slot.
template <int CtaGroup>
__device__ __forceinline__ void tmem_alloc(uint32_t *smem_slot, uint32_t ncols)
{
    if constexpr (CtaGroup == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         smem_u32(smem_slot)),
                     "r"(ncols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    } else {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         smem_u32(smem_slot)),
                     "r"(ncols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
}

template <int CtaGroup>
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols)
{
    if constexpr (CtaGroup == 1)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr),
                     "r"(ncols)
                     : "memory");
    else
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr),
                     "r"(ncols)
                     : "memory");
}

// 32 lanes x 32 consecutive 32-bit columns -> 32 registers per thread.
// Thread t of the warp reads TMEM lane (lane field of taddr) + t.
__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
          "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
          "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}

__device__ __forceinline__ void tmem_ld_wait()
{
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// 32 lanes x 1 column store (one register per thread); used to place sparse
// metadata and scale factors into TMEM from registers.
__device__ __forceinline__ void tmem_st_32x32b_x1(uint32_t taddr, uint32_t v)
{
    asm volatile("tcgen05.st.sync.aligned.32x32b.x1.b32 [%0], {%1};" ::"r"(taddr), "r"(v)
                 : "memory");
}

__device__ __forceinline__ void tmem_st_wait()
{
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// Shared memory -> TMEM copy of 32 rows x 128 bits replicated to the four
// 32-lane quarters (the scale-factor staging shape).
template <int CtaGroup>
__device__ __forceinline__ void tmem_cp_32x128b_warpx4(uint32_t taddr, uint64_t smem_desc)
{
    if constexpr (CtaGroup == 1)
        asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr),
                     "l"(smem_desc)
                     : "memory");
    else
        asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(taddr),
                     "l"(smem_desc)
                     : "memory");
}

// 128 rows x 128 bits (lane i <- row i).
template <int CtaGroup>
__device__ __forceinline__ void tmem_cp_128x128b(uint32_t taddr, uint64_t smem_desc)
{
    if constexpr (CtaGroup == 1)
        asm volatile("tcgen05.cp.cta_group::1.128x128b [%0], %1;" ::"r"(taddr), "l"(smem_desc)
                     : "memory");
    else
        asm volatile("tcgen05.cp.cta_group::2.128x128b [%0], %1;" ::"r"(taddr), "l"(smem_desc)
                     : "memory");
}

// 128 rows x 256 bits (lane i <- row i, eight columns).
template <int CtaGroup>
__device__ __forceinline__ void tmem_cp_128x256b(uint32_t taddr, uint64_t smem_desc)
{
    if constexpr (CtaGroup == 1)
        asm volatile("tcgen05.cp.cta_group::1.128x256b [%0], %1;" ::"r"(taddr), "l"(smem_desc)
                     : "memory");
    else
        asm volatile("tcgen05.cp.cta_group::2.128x256b [%0], %1;" ::"r"(taddr), "l"(smem_desc)
                     : "memory");
}

// ---- tcgen05.commit ------------------------------------------------------------------

// All prior tcgen05 async ops of this thread arrive (count 1) on `bar` when done.
__device__ __forceinline__ void tc_commit(uint64_t *bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                     smem_u32(bar))
                 : "memory");
}

// CTA-pair form: arrives on the barrier at this offset in every CTA of `cta_mask`.
__device__ __forceinline__ void tc_commit_pair(uint64_t *bar, uint16_t cta_mask)
{
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 "
        "[%0], %1;" ::"r"(smem_u32(bar)),
        "h"(cta_mask)
        : "memory");
}

// ---- descriptors -----------------------------------------------------------------------

// 64-bit shared-memory matrix descriptor (sm_100 "version 1" encoding):
//   [0,14)  start address >> 4         [16,30) leading-dimension byte offset >> 4
//   [32,46) stride-dimension byte offset >> 4      [46,48) version = 1
//   [49,52) base offset                [61,64) swizzle: 0 none, 2 128B, 4 64B, 6 32B
// K-major operands: SBO is the distance between consecutive 8-row groups; LBO
// is the distance between the two 16-byte K chunks of one MMA when there is no
// swizzle (with a swizzle the chunks are adjacent inside the swizzled row).
enum : uint32_t { kSwizzleNone = 0, kSwizzle128B = 2, kSwizzle64B = 4, kSwizzle32B = 6 };

__host__ __device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr, uint32_t lbo_bytes,
                                                            uint32_t sbo_bytes, uint32_t swizzle)
{
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)(swizzle & 7) << 61;
    return d;
}

// 32-bit instruction descriptor for kind::f16 / tf32 / f8f6f4 / i8:
//   [0,2) sparse id2  [2] sparse  [3] saturate  [4,6) D format (0 f16, 1 f32, 2 s32)
//   [7,10) A format   [10,13) B format   [13] negate A  [14] negate B
//   [15] A major (0 = K)  [16] B major (0 = K)  [17,23) N>>3  [24,29) M>>4
enum : uint32_t {
    kFmtF16 = 0, kFmtBF16 = 1, kFmtTF32 = 2,      // kind::f16 / kind::tf32
    kFmtE4M3 = 0, kFmtE5M2 = 1, kFmtE2M1x8 = 5,   // kind::f8f6f4
    kFmtU8 = 0, kFmtS8 = 1,                       // kind::i8
    kFmtE2M1 = 1,                                 // kind::mxf4 / mxf4nvf4
    kAccF16 = 0, kAccF32 = 1, kAccS32 = 2
};

__host__ __device__ __forceinline__ uint32_t make_idesc(uint32_t m, uint32_t n, uint32_t a_fmt,
                                                        uint32_t b_fmt, uint32_t acc_fmt,
                                                        bool sparse = false)
{
    uint32_t d = 0;
    d |= (sparse ? 1u : 0u) << 2;
    d |= (acc_fmt & 3u) << 4;
    d |= (a_fmt & 7u) << 7;
    d |= (b_fmt & 7u) << 10;
    d |= ((n >> 3) & 0x3Fu) << 17;
    d |= ((m >> 4) & 0x1Fu) << 24;
    return d;
}

// Block-scaled kinds (mxf8f6f4 / mxf4 / mxf4nvf4): same operand fields, plus
//   [4,6) B scale-factor id   [23] scale format (0 ue4m3, 1 ue8m0)
//   [29,31) A scale-factor id [31] K size selector (0 = the dense K64 / sparse K128 shape)
__host__ __device__ __forceinline__ uint32_t make_idesc_block_scaled(uint32_t m, uint32_t n,
                                                                     uint32_t a_fmt, uint32_t b_fmt,
                                                                     uint32_t scale_fmt,
                                                                     uint32_t a_sf_id,
                                                                     uint32_t b_sf_id,
                                                                     bool sparse = false)
{
    uint32_t d = 0;
    d |= (sparse ? 1u : 0u) << 2;
    d |= (b_sf_id & 3u) << 4;
    d |= (a_fmt & 7u) << 7;
    d |= (b_fmt & 7u) << 10;
    d |= ((n >> 3) & 0x3Fu) << 17;
    d |= (scale_fmt & 1u) << 23;
    d |= ((m >> 4) & 0x1Fu) << 24;
    d |= (a_sf_id & 3u) << 29;
    return d;
}

// ---- tcgen05.mma ---------------------------------------------------------------------------

#define CLPK_DEFINE_MMA_SS(NAME, KINDSTR)                                                        \
    __device__ __forceinline__ void NAME(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,      \
                                         uint32_t idesc, uint32_t accumulate)                    \
    {                                                                                            \
        asm volatile(                                                                            \
            "{\n\t"                                                                              \
            ".reg .pred p;\n\t"                                                                  \
            "setp.ne.b32 p, %4, 0;\n\t"                                                          \
            "tcgen05.mma.cta_group::1." KINDSTR " [%0], %1, %2, %3, p;\n\t"                      \
            "}\n" ::"r"(d_tmem),                                                                 \
            "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)                                \
            : "memory");                                                                         \
    }

CLPK_DEFINE_MMA_SS(mma_f16_ss, "kind::f16")
CLPK_DEFINE_MMA_SS(mma_tf32_ss, "kind::tf32")
CLPK_DEFINE_MMA_SS(mma_f8f6f4_ss, "kind::f8f6f4")
CLPK_DEFINE_MMA_SS(mma_i8_ss, "kind::i8")

#define CLPK_DEFINE_MMA2_SS(NAME, KINDSTR)                                                       \
    __device__ __forceinline__ void NAME(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,      \
                                         uint32_t idesc, uint32_t accumulate)                    \
    {                                                                                            \
        asm volatile(                                                                            \
            "{\n\t"                                                                              \
            ".reg .pred p;\n\t"                                                                  \
            "setp.ne.b32 p, %4, 0;\n\t"                                                          \
            "tcgen05.mma.cta_group::2." KINDSTR " [%0], %1, %2, %3, p;\n\t"                      \
            "}\n" ::"r"(d_tmem),                                                                 \
            "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)                                \
            : "memory");                                                                         \
    }

CLPK_DEFINE_MMA2_SS(mma2_f16_ss, "kind::f16")
CLPK_DEFINE_MMA2_SS(mma2_f8f6f4_ss, "kind::f8f6f4")
CLPK_DEFINE_MMA2_SS(mma2_tf32_ss, "kind::tf32")
CLPK_DEFINE_MMA2_SS(mma2_i8_ss, "kind::i8")

// Block-scaled: scale factors for A and B live in TMEM.
#define CLPK_DEFINE_MMA_BS(NAME, CTAGROUP, KINDSTR)                                              \
    __device__ __forceinline__ void NAME(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,      \
                                         uint32_t idesc, uint32_t sfa_tmem, uint32_t sfb_tmem,   \
                                         uint32_t accumulate)                                    \
    {                                                                                            \
        asm volatile(                                                                            \
            "{\n\t"                                                                              \
            ".reg .pred p;\n\t"                                                                  \
            "setp.ne.b32 p, %4, 0;\n\t"                                                          \
            "tcgen05.mma.cta_group::" CTAGROUP "." KINDSTR " [%0], %1, %2, %3, [%5], [%6], p;\n\t" \
            "}\n" ::"r"(d_tmem),                                                                 \
            "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)  \
            : "memory");                                                                         \
    }

CLPK_DEFINE_MMA_BS(mma_mxf4_bs, "1", "kind::mxf4.block_scale.scale_vec::2X")
CLPK_DEFINE_MMA_BS(mma_nvf4_bs, "1", "kind::mxf4nvf4.block_scale.scale_vec::4X")
CLPK_DEFINE_MMA_BS(mma2_nvf4_bs, "2", "kind::mxf4nvf4.block_scale.scale_vec::4X")
CLPK_DEFINE_MMA_BS(mma2_mxf4_bs, "2", "kind::mxf4.block_scale.scale_vec::2X")

// 2:4 sparse A: metadata lives in TMEM.
#define CLPK_DEFINE_MMA_SP(NAME, CTAGROUP, KINDSTR)                                              \
    __device__ __forceinline__ void NAME(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,      \
                                         uint32_t idesc, uint32_t meta_tmem, uint32_t accumulate) \
    {                                                                                            \
        asm volatile(                                                                            \
            "{\n\t"                                                                              \
            ".reg .pred p;\n\t"                                                                  \
            "setp.ne.b32 p, %4, 0;\n\t"                                                          \
            "tcgen05.mma.sp.cta_group::" CTAGROUP "." KINDSTR " [%0], %1, %2, [%5], %3, p;\n\t"  \
            "}\n" ::"r"(d_tmem),                                                                 \
            "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(meta_tmem)                \
            : "memory");                                                                         \
    }

CLPK_DEFINE_MMA_SP(mma_f16_sp, "1", "kind::f16")
CLPK_DEFINE_MMA_SP(mma_f8f6f4_sp, "1", "kind::f8f6f4")
CLPK_DEFINE_MMA_SP(mma_i8_sp, "1", "kind::i8")
CLPK_DEFINE_MMA_SP(mma2_f8f6f4_sp, "2", "kind::f8f6f4")
CLPK_DEFINE_MMA_SP(mma2_i8_sp, "2", "kind::i8")

#define CLPK_DEFINE_MMA_SP_BS(NAME, CTAGROUP, KINDSTR)                                           \
    __device__ __forceinline__ void NAME(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,      \
                                         uint32_t idesc, uint32_t meta_tmem, uint32_t sfa_tmem,  \
                                         uint32_t sfb_tmem, uint32_t accumulate)                 \
    {                                                                                            \
        asm volatile(                                                                            \
            "{\n\t"                                                                              \
            ".reg .pred p;\n\t"                                                                  \
            "setp.ne.b32 p, %4, 0;\n\t"                                                          \
            "tcgen05.mma.sp.cta_group::" CTAGROUP "." KINDSTR " [%0], %1, %2, [%7], %3, [%5], [%6], p;\n\t" \
            "}\n" ::"r"(d_tmem),                                                                 \
            "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem), \
            "r"(meta_tmem)                                                                       \
            : "memory");                                                                         \
    }

CLPK_DEFINE_MMA_SP_BS(mma_mxf4_sp_bs, "1", "kind::mxf4.block_scale.scale_vec::2X")
CLPK_DEFINE_MMA_SP_BS(mma_nvf4_sp_bs, "1", "kind::mxf4nvf4.block_scale.scale_vec::4X")
CLPK_DEFINE_MMA_SP_BS(mma2_mxf4_sp_bs, "2", "kind::mxf4.block_scale.scale_vec::2X")
CLPK_DEFINE_MMA_SP_BS(mma2_nvf4_sp_bs, "2", "kind::mxf4nvf4.block_scale.scale_vec::4X")

} // namespace clpk
