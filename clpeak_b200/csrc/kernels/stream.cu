// Global-memory bandwidth kernels.
//
//  * global_bandwidth_v<W>: the reference read-and-sum test with its exact
//    per-thread order (16 fetches at a 256-element stride inside a block-owned
//    region), widened to 64-bit indexing so buffers beyond 4 Gi elements work.
//  * stream read / copy / triad in two flavours:
//      LDG - persistent grid, four independent 128-bit loads per thread per
//            step (streaming cache hints), registers in between;
//      TMA - one elected thread per CTA moves 32 KiB tiles with
//            cp.async.bulk through a ring of shared-memory stages; copy never
//            touches registers, triad computes in place in shared memory.
//
// HBM traffic per pass (the algorithmic bytes the roofline is computed from):
// read n, copy 2n, triad 3n bytes for n-byte arrays; GPUs do not
// write-allocate, so these are the true DRAM bytes.
#include <atomic>
#include <mutex>

#include "../clpk_internal.h"
#include "../clpk_ptx.cuh"

namespace clpk {

constexpr int kFetchPerWI = 16;   // FETCH_PER_WI of the reference (include/common/common.h:56)

template <typename V>
__device__ __forceinline__ float lane_sum(const V &v);
template <>
__device__ __forceinline__ float lane_sum<float>(const float &v) { return v; }
template <>
__device__ __forceinline__ float lane_sum<float2>(const float2 &v) { return v.x + v.y; }
template <>
__device__ __forceinline__ float lane_sum<float4>(const float4 &v)
{
    return v.x + v.y + v.z + v.w;   // ((x + y) + z) + w
}

__device__ __forceinline__ void vadd(float &a, const float &b) { a += b; }
__device__ __forceinline__ void vadd(float2 &a, const float2 &b) { a.x += b.x; a.y += b.y; }
__device__ __forceinline__ void vadd(float4 &a, const float4 &b)
{
    a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
}

template <typename V>
__global__ void __launch_bounds__(256) global_bandwidth_kernel(const V *__restrict__ in,
                                                               float *__restrict__ out)
{
    const uint64_t gid = (uint64_t)blockIdx.x * 256 + threadIdx.x;
    uint64_t offset = (uint64_t)blockIdx.x * 256 * kFetchPerWI + threadIdx.x;
    V vals[kFetchPerWI];
#pragma unroll
    for (int i = 0; i < kFetchPerWI; i++)
        vals[i] = __ldg(in + offset + (uint64_t)i * 256);
    V sum{};
#pragma unroll
    for (int i = 0; i < kFetchPerWI; i++)
        vadd(sum, vals[i]);
    out[gid] = lane_sum(sum);
}

// ---- LDG flavour ---------------------------------------------------------------------

constexpr int kLdgThreads = 512;
constexpr int kLdgUnroll = 4;
constexpr int kLdgCtasPerSm = 4;

__device__ __forceinline__ uint32_t xor4(const uint4 &v) { return v.x ^ v.y ^ v.z ^ v.w; }

__device__ __forceinline__ void cta_xor_store(uint32_t x, uint32_t *slot)
{
    __shared__ uint32_t warp_x[32];
    for (int o = 16; o > 0; o >>= 1)
        x ^= __shfl_xor_sync(0xffffffffu, x, o);
    if ((threadIdx.x & 31) == 0)
        warp_x[threadIdx.x >> 5] = x;
    __syncthreads();
    if (threadIdx.x < 32) {
        uint32_t y = threadIdx.x < (blockDim.x >> 5) ? warp_x[threadIdx.x] : 0u;
        for (int o = 16; o > 0; o >>= 1)
            y ^= __shfl_xor_sync(0xffffffffu, y, o);
        if (threadIdx.x == 0)
            *slot = y;
    }
}

__global__ void __launch_bounds__(kLdgThreads) stream_read_ldg(const uint4 *__restrict__ src,
                                                               uint64_t n16,
                                                               uint32_t *__restrict__ partials)
{
    constexpr uint64_t kTile = (uint64_t)kLdgThreads * kLdgUnroll;
    uint32_t acc = 0;
    const uint64_t n_full = n16 / kTile;
    for (uint64_t t = blockIdx.x; t < n_full; t += gridDim.x) {
        const uint4 *p = src + t * kTile + threadIdx.x;
        uint4 v[kLdgUnroll];
#pragma unroll
        for (int u = 0; u < kLdgUnroll; u++)
            v[u] = __ldcs(p + u * kLdgThreads);
#pragma unroll
        for (int u = 0; u < kLdgUnroll; u++)
            acc ^= xor4(v[u]);
    }
    if (blockIdx.x == 0) {
        for (uint64_t i = n_full * kTile + threadIdx.x; i < n16; i += kLdgThreads)
            acc ^= xor4(__ldcs(src + i));
    }
    cta_xor_store(acc, partials + blockIdx.x);
}

__global__ void __launch_bounds__(kLdgThreads) stream_copy_ldg(uint4 *__restrict__ dst,
                                                               const uint4 *__restrict__ src,
                                                               uint64_t n16)
{
    constexpr uint64_t kTile = (uint64_t)kLdgThreads * kLdgUnroll;
    const uint64_t n_full = n16 / kTile;
    for (uint64_t t = blockIdx.x; t < n_full; t += gridDim.x) {
        const uint64_t base = t * kTile + threadIdx.x;
        uint4 v[kLdgUnroll];
#pragma unroll
        for (int u = 0; u < kLdgUnroll; u++)
            v[u] = __ldcs(src + base + u * kLdgThreads);
#pragma unroll
        for (int u = 0; u < kLdgUnroll; u++)
            __stcs(dst + base + u * kLdgThreads, v[u]);
    }
    if (blockIdx.x == 0) {
        for (uint64_t i = n_full * kTile + threadIdx.x; i < n16; i += kLdgThreads)
            __stcs(dst + i, __ldcs(src + i));
    }
}

__device__ __forceinline__ float4 triad4(const float4 &b, const float4 &c, float s)
{
    // b + s*c as two roundings (multiply, then add): no FMA contraction, so the
    // host check can use plain C arithmetic.
    return make_float4(__fadd_rn(b.x, __fmul_rn(s, c.x)), __fadd_rn(b.y, __fmul_rn(s, c.y)),
                       __fadd_rn(b.z, __fmul_rn(s, c.z)), __fadd_rn(b.w, __fmul_rn(s, c.w)));
}

__global__ void __launch_bounds__(kLdgThreads) stream_triad_ldg(float4 *__restrict__ a,
                                                                const float4 *__restrict__ b,
                                                                const float4 *__restrict__ c,
                                                                float s, uint64_t n4,
                                                                uint64_t n_tail_floats)
{
    constexpr int kU = 2;   // two b + two c loads in flight per thread
    constexpr uint64_t kTile = (uint64_t)kLdgThreads * kU;
    const uint64_t n_full = n4 / kTile;
    for (uint64_t t = blockIdx.x; t < n_full; t += gridDim.x) {
        const uint64_t base = t * kTile + threadIdx.x;
        float4 vb[kU], vc[kU];
#pragma unroll
        for (int u = 0; u < kU; u++) {
            vb[u] = __ldcs(b + base + u * kLdgThreads);
            vc[u] = __ldcs(c + base + u * kLdgThreads);
        }
#pragma unroll
        for (int u = 0; u < kU; u++)
            __stcs(a + base + u * kLdgThreads, triad4(vb[u], vc[u], s));
    }
    if (blockIdx.x == 0) {
        for (uint64_t i = n_full * kTile + threadIdx.x; i < n4; i += kLdgThreads)
            __stcs(a + i, triad4(__ldcs(b + i), __ldcs(c + i), s));
        // floats beyond the last whole float4
        const float *bf = reinterpret_cast<const float *>(b) + n4 * 4;
        const float *cf = reinterpret_cast<const float *>(c) + n4 * 4;
        float *af = reinterpret_cast<float *>(a) + n4 * 4;
        if (threadIdx.x < n_tail_floats)
            af[threadIdx.x] = __fadd_rn(bf[threadIdx.x], __fmul_rn(s, cf[threadIdx.x]));
    }
}

// ---- TMA (cp.async.bulk) flavour ------------------------------------------------------------
//
// Shared memory: kTmaStages stages of kTmaTile bytes (triad: two tiles per
// stage), then the barriers.  Tiles are handed out round-robin:
// CTA b owns tiles b, b+grid, b+2*grid, ...

// ---- 256-bit accesses, one 8 KiB tile per CTA ---------------------------------------------
//
// The fastest form measured on B200: 256 threads, each moving one 32-byte vector
// (ld/st.global.v4.b64, new with sm_100), and as many CTAs as there are tiles.  The
// hardware block scheduler hands tiles out in address order as SMs free up, so at any
// moment the whole chip works inside a window of a few MiB and HBM pages are opened once
// per direction.  A persistent grid with a fixed tile-to-CTA map loses that as its CTAs
// drift apart: copy 6.25 -> 6.95 TB/s, read 7.2 -> 7.6, triad 6.55 -> 7.1 (8 GiB arrays).
// L1::no_allocate + L2::evict_first: nothing is read twice.
constexpr int kWideThreads = 256;
constexpr uint64_t kWideTileBytes = (uint64_t)kWideThreads * 32;
constexpr int kWideSlots = 4096;                 // checksum partials of the read kernel

struct __align__(32) Vec32 {
    unsigned long long a, b, c, d;
};

__device__ __forceinline__ Vec32 ld_stream32(const Vec32 *p)
{
    Vec32 v;
    asm volatile("ld.global.L1::no_allocate.L2::evict_first.v4.b64 {%0, %1, %2, %3}, [%4];"
                 : "=l"(v.a), "=l"(v.b), "=l"(v.c), "=l"(v.d)
                 : "l"(p));
    return v;
}

__device__ __forceinline__ void st_stream32(Vec32 *p, const Vec32 &v)
{
    asm volatile("st.global.L1::no_allocate.L2::evict_first.v4.b64 [%0], {%1, %2, %3, %4};" ::"l"(p), "l"(v.a),
                 "l"(v.b), "l"(v.c), "l"(v.d)
                 : "memory");
}

// n_tiles full tiles, one per CTA; CTA 0 also takes the tail of n_tail16 16-byte pieces.
__global__ void __launch_bounds__(kWideThreads) stream_read_wide(const Vec32 *__restrict__ src, uint64_t n_tiles,
                                                                 uint64_t n_tail16, uint32_t *__restrict__ slots)
{
    unsigned long long x = 0;
    if (blockIdx.x < n_tiles) {
        const Vec32 v = ld_stream32(src + (uint64_t)blockIdx.x * kWideThreads + threadIdx.x);
        x = v.a ^ v.b ^ v.c ^ v.d;
    }
    uint32_t y = (uint32_t)x ^ (uint32_t)(x >> 32);
    if (blockIdx.x == 0) {
        const uint4 *tail = reinterpret_cast<const uint4 *>(src + n_tiles * kWideThreads);
        for (uint64_t i = threadIdx.x; i < n_tail16; i += kWideThreads)
            y ^= xor4(__ldcs(tail + i));
    }
    for (int o = 16; o > 0; o >>= 1)
        y ^= __shfl_xor_sync(0xffffffffu, y, o);
    __shared__ uint32_t warp_x[kWideThreads / 32];
    if ((threadIdx.x & 31) == 0)
        warp_x[threadIdx.x >> 5] = y;
    __syncthreads();
    if (threadIdx.x == 0) {
        uint32_t z = 0;
#pragma unroll
        for (int i = 0; i < kWideThreads / 32; i++)
            z ^= warp_x[i];
        atomicXor(slots + (blockIdx.x & (kWideSlots - 1)), z);       // XOR: the order does not matter
    }
}

__global__ void __launch_bounds__(kWideThreads) stream_copy_wide(Vec32 *__restrict__ dst, const Vec32 *__restrict__ src,
                                                                 uint64_t n_tiles, uint64_t n_tail16)
{
    if (blockIdx.x < n_tiles) {
        const uint64_t i = (uint64_t)blockIdx.x * kWideThreads + threadIdx.x;
        st_stream32(dst + i, ld_stream32(src + i));
    }
    if (blockIdx.x == 0) {
        const uint4 *ts = reinterpret_cast<const uint4 *>(src + n_tiles * kWideThreads);
        uint4 *td = reinterpret_cast<uint4 *>(dst + n_tiles * kWideThreads);
        for (uint64_t i = threadIdx.x; i < n_tail16; i += kWideThreads)
            __stcs(td + i, __ldcs(ts + i));
    }
}

constexpr uint32_t kTmaTile = 32768;
constexpr int kTmaStages = 6;
constexpr int kTmaTriadStages = 3;
constexpr uint32_t kTmaTriadTile = 32768;

__device__ __forceinline__ uint32_t tile_bytes(uint64_t tile, uint64_t n_bytes, uint32_t tile_sz)
{
    const uint64_t off = tile * tile_sz;
    const uint64_t left = n_bytes - off;
    return left < tile_sz ? (uint32_t)left : tile_sz;
}

// status word: 0 ok, otherwise 1 + id of the wait that expired.
__device__ __forceinline__ void report_timeout(uint32_t *status, uint32_t where)
{
    atomicCAS(status, 0u, 1u + where);
}

// Tiles are claimed from a per-launch counter rather than dealt out round-robin, so the chip
// as a whole walks the array in address order whatever the relative speed of the SMs (a
// fixed tile-to-CTA map lets the CTAs drift apart and costs about 10 % of the bandwidth).
// The producer leaves each stage's byte count in shared memory; a count of zero ends the
// consumers' loop.
__global__ void __launch_bounds__(160) stream_read_tma(const uint8_t *__restrict__ src,
                                                       uint64_t n_bytes,
                                                       uint32_t *__restrict__ partials,
                                                       uint32_t *__restrict__ status,
                                                       unsigned long long *__restrict__ next_tile)
{
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t *full = reinterpret_cast<uint64_t *>(smem + (size_t)kTmaStages * kTmaTile);
    uint64_t *empty = full + kTmaStages;
    volatile uint32_t *stage_bytes = reinterpret_cast<volatile uint32_t *>(empty + kTmaStages);
    const uint64_t n_tiles = (n_bytes + kTmaTile - 1) / kTmaTile;
    const int warp = threadIdx.x >> 5;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kTmaStages; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 4);   // one arrive per consumer warp
        }
        mbar_fence_init();
    }
    __syncthreads();

    uint32_t acc = 0;
    if (warp == 0) {
        if (threadIdx.x == 0) {
            for (uint32_t j = 0;; j++) {
                const int s = j % kTmaStages;
                const uint32_t round = j / kTmaStages;
                if (round > 0 && !mbar_wait(&empty[s], (round - 1) & 1)) {
                    report_timeout(status, 0);
                    break;
                }
                const uint64_t t = atomicAdd(next_tile, 1ull);
                if (t >= n_tiles) {
                    stage_bytes[s] = 0;
                    mbar_arrive(&full[s]);
                    break;
                }
                const uint32_t bytes = tile_bytes(t, n_bytes, kTmaTile);
                stage_bytes[s] = bytes;
                mbar_expect_tx(&full[s], bytes);
                bulk_g2s(smem + (size_t)s * kTmaTile, src + t * kTmaTile, bytes, &full[s]);
            }
        }
    } else {
        const int ctid = threadIdx.x - 32;   // 0..127
        for (uint32_t j = 0;; j++) {
            const int s = j % kTmaStages;
            const uint32_t round = j / kTmaStages;
            if (!mbar_wait(&full[s], round & 1)) {
                report_timeout(status, 1);
                break;
            }
            const uint32_t n16 = stage_bytes[s] / 16;
            if (n16 == 0)
                break;
            const uint4 *p = reinterpret_cast<const uint4 *>(smem + (size_t)s * kTmaTile);
            for (uint32_t i = ctid; i < n16; i += 128)
                acc ^= xor4(p[i]);
            __syncwarp();
            if ((threadIdx.x & 31) == 0)
                mbar_arrive(&empty[s]);
        }
    }
    cta_xor_store(acc, partials + blockIdx.x);
}

__global__ void __launch_bounds__(32) stream_copy_tma(uint8_t *__restrict__ dst,
                                                      const uint8_t *__restrict__ src,
                                                      uint64_t n_bytes,
                                                      uint32_t *__restrict__ status,
                                                      unsigned long long *__restrict__ next_tile)
{
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t *full = reinterpret_cast<uint64_t *>(smem + (size_t)kTmaStages * kTmaTile);
    const uint64_t n_tiles = (n_bytes + kTmaTile - 1) / kTmaTile;
    if (threadIdx.x != 0)
        return;
    for (int s = 0; s < kTmaStages; s++)
        mbar_init(&full[s], 1);
    mbar_fence_init();

    // tiles claimed in address order, as in stream_read_tma
    uint64_t tile_of[kTmaStages];
    uint64_t issued = 0;
    bool more = true;
    auto issue_load = [&]() {
        const uint64_t t = atomicAdd(next_tile, 1ull);
        if (t >= n_tiles) {
            more = false;
            return;
        }
        const int s = (int)(issued % kTmaStages);
        tile_of[s] = t;
        const uint32_t bytes = tile_bytes(t, n_bytes, kTmaTile);
        mbar_expect_tx(&full[s], bytes);
        bulk_g2s(smem + (size_t)s * kTmaTile, src + t * kTmaTile, bytes, &full[s]);
        issued++;
    };
    for (int i = 0; i < kTmaStages && more; i++)
        issue_load();
    for (uint64_t j = 0; j < issued; j++) {
        const int s = (int)(j % kTmaStages);
        const uint64_t t = tile_of[s];
        if (!mbar_wait(&full[s], (uint32_t)(j / kTmaStages) & 1)) {
            report_timeout(status, 2);
            break;
        }
        bulk_s2g(dst + t * kTmaTile, smem + (size_t)s * kTmaTile, tile_bytes(t, n_bytes, kTmaTile));
        bulk_commit();
        // Store j-1 has finished reading its stage once at most one group is
        // still pending; that stage can take the next tile.
        bulk_wait_read<1>();
        if (j >= 1 && more)
            issue_load();
    }
    bulk_wait<0>();
}

__global__ void __launch_bounds__(kWideThreads) stream_triad_wide(Vec32 *__restrict__ a, const Vec32 *__restrict__ b,
                                                                  const Vec32 *__restrict__ c, float s,
                                                                  uint64_t n_tiles, uint64_t n_tail_floats)
{
    if (blockIdx.x < n_tiles) {
        const uint64_t i = (uint64_t)blockIdx.x * kWideThreads + threadIdx.x;
        Vec32 vb = ld_stream32(b + i);
        const Vec32 vc = ld_stream32(c + i);
        float4 *fb = reinterpret_cast<float4 *>(&vb);
        const float4 *fc = reinterpret_cast<const float4 *>(&vc);
        fb[0] = triad4(fb[0], fc[0], s);
        fb[1] = triad4(fb[1], fc[1], s);
        st_stream32(a + i, vb);
    }
    if (blockIdx.x == 0) {
        const float *tb = reinterpret_cast<const float *>(b + n_tiles * kWideThreads);
        const float *tc = reinterpret_cast<const float *>(c + n_tiles * kWideThreads);
        float *ta = reinterpret_cast<float *>(a + n_tiles * kWideThreads);
        for (uint64_t i = threadIdx.x; i < n_tail_floats; i += kWideThreads)
            ta[i] = __fadd_rn(tb[i], __fmul_rn(s, tc[i]));
    }
}

__global__ void __launch_bounds__(192) stream_triad_tma(float *__restrict__ a,
                                                        const float *__restrict__ b,
                                                        const float *__restrict__ c, float s,
                                                        uint64_t n_bytes,
                                                        uint32_t *__restrict__ status,
                                                        unsigned long long *__restrict__ next_tile)
{
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr uint32_t kStage = 2 * kTmaTriadTile;
    uint64_t *full = reinterpret_cast<uint64_t *>(smem + (size_t)kTmaTriadStages * kStage);
    uint64_t *done = full + kTmaTriadStages;
    uint64_t *empty = done + kTmaTriadStages;
    // per stage: the claimed tile's index and byte count (0 bytes = no more tiles)
    volatile uint64_t *stage_tile = reinterpret_cast<volatile uint64_t *>(empty + kTmaTriadStages);
    volatile uint32_t *stage_bytes = reinterpret_cast<volatile uint32_t *>(const_cast<uint64_t *>(stage_tile) + kTmaTriadStages);
    const uint64_t n_tiles = (n_bytes + kTmaTriadTile - 1) / kTmaTriadTile;
    const int warp = threadIdx.x >> 5;

    if (threadIdx.x == 0) {
        for (int i = 0; i < kTmaTriadStages; i++) {
            mbar_init(&full[i], 1);
            mbar_init(&done[i], 4);
            mbar_init(&empty[i], 1);
        }
        mbar_fence_init();
    }
    __syncthreads();

    const uint8_t *bb = reinterpret_cast<const uint8_t *>(b);
    const uint8_t *cb = reinterpret_cast<const uint8_t *>(c);
    uint8_t *ab = reinterpret_cast<uint8_t *>(a);

    if (warp == 0) {
        if (threadIdx.x == 0) {
            for (uint32_t j = 0;; j++) {
                const int st = j % kTmaTriadStages;
                const uint32_t round = j / kTmaTriadStages;
                if (round > 0 && !mbar_wait(&empty[st], (round - 1) & 1)) {
                    report_timeout(status, 3);
                    break;
                }
                const uint64_t t = atomicAdd(next_tile, 1ull);
                if (t >= n_tiles) {
                    stage_bytes[st] = 0;
                    mbar_arrive(&full[st]);
                    break;
                }
                const uint32_t bytes = tile_bytes(t, n_bytes, kTmaTriadTile);
                stage_tile[st] = t;
                stage_bytes[st] = bytes;
                uint8_t *sb = smem + (size_t)st * kStage;
                mbar_expect_tx(&full[st], 2 * bytes);
                bulk_g2s(sb, bb + t * kTmaTriadTile, bytes, &full[st]);
                bulk_g2s(sb + kTmaTriadTile, cb + t * kTmaTriadTile, bytes, &full[st]);
            }
        }
    } else if (warp <= 4) {
        const int ctid = threadIdx.x - 32;
        for (uint32_t j = 0;; j++) {
            const int st = j % kTmaTriadStages;
            if (!mbar_wait(&full[st], (j / kTmaTriadStages) & 1)) {
                report_timeout(status, 4);
                break;
            }
            const uint32_t n4 = stage_bytes[st] / 16;
            if (n4 != 0) {
                float4 *pb = reinterpret_cast<float4 *>(smem + (size_t)st * kStage);
                const float4 *pc = reinterpret_cast<const float4 *>(smem + (size_t)st * kStage + kTmaTriadTile);
                for (uint32_t i = ctid; i < n4; i += 128)
                    pb[i] = triad4(pb[i], pc[i], s);
                fence_proxy_async_smem();
            }
            __syncwarp();
            if ((threadIdx.x & 31) == 0)
                mbar_arrive(&done[st]);        // also for the end marker: the store thread must see it
            if (n4 == 0)
                break;
        }
    } else {
        if (threadIdx.x == 160) {
            for (uint32_t j = 0;; j++) {
                const int st = j % kTmaTriadStages;
                if (!mbar_wait(&done[st], (j / kTmaTriadStages) & 1)) {
                    report_timeout(status, 5);
                    break;
                }
                const uint32_t bytes = stage_bytes[st];
                if (bytes == 0)
                    break;
                bulk_s2g(ab + stage_tile[st] * kTmaTriadTile, smem + (size_t)st * kStage, bytes);
                bulk_commit();
                bulk_wait_read<0>();
                mbar_arrive(&empty[st]);
            }
            bulk_wait<0>();
        }
    }
}

// Per-device status word for the TMA kernels (timeouts are reported through
// the return code of the *next* synchronising call via clpk_stream_status()).
static uint32_t *g_status[64] = {nullptr};
static std::mutex g_lazy_mutex;          // first use of a device by two host threads at once allocates once

static int status_word(uint32_t **out)
{
    int dev = 0;
    CLPK_CUDA(cudaGetDevice(&dev));
    CLPK_REQUIRE(dev >= 0 && dev < 64, "device ordinal %d out of range", dev);
    std::lock_guard<std::mutex> lk(g_lazy_mutex);
    if (!g_status[dev]) {
        uint32_t *w = nullptr;
        CLPK_CUDA(cudaMalloc(&w, sizeof(uint32_t)));
        CLPK_CUDA(cudaMemset(w, 0, sizeof(uint32_t)));
        g_status[dev] = w;
    }
    *out = g_status[dev];
    return CLPK_OK;
}

static int read_grid(int variant)
{
    if (variant == CLPK_STREAM_WIDE)
        return kWideSlots;
    return variant == CLPK_STREAM_TMA ? num_sms() : num_sms() * kLdgCtasPerSm;
}

static bool known_variant(int v) { return v == CLPK_STREAM_LDG || v == CLPK_STREAM_TMA || v == CLPK_STREAM_WIDE; }

// Launch geometry of the one-tile-per-CTA kernels: at least one CTA (it owns the tail).
static unsigned wide_grid(uint64_t n_tiles)
{
    return (unsigned)(n_tiles ? n_tiles : 1);
}

constexpr size_t kTmaSmem = (size_t)kTmaStages * kTmaTile + 2 * kTmaStages * sizeof(uint64_t) + kTmaStages * sizeof(uint32_t);
constexpr size_t kTmaTriadSmem =
    (size_t)kTmaTriadStages * 2 * kTmaTriadTile + 4 * kTmaTriadStages * sizeof(uint64_t) + kTmaTriadStages * sizeof(uint32_t);

// Tile counters of the TMA kernels: one 8-byte counter per launch out of a per-device ring
// (launches on different streams get different ones), zeroed in stream order before the kernel.
constexpr int kCounterRing = 32;
static unsigned long long *g_counters[64] = {nullptr};
static std::atomic<unsigned> g_next_counter{0};

static int tile_counter(cudaStream_t s, unsigned long long **out)
{
    int dev = 0;
    CLPK_CUDA(cudaGetDevice(&dev));
    CLPK_REQUIRE(dev >= 0 && dev < 64, "device ordinal %d out of range", dev);
    {
        std::lock_guard<std::mutex> lk(g_lazy_mutex);
        if (!g_counters[dev])
            CLPK_CUDA(cudaMalloc(&g_counters[dev], kCounterRing * sizeof(unsigned long long)));
    }
    *out = g_counters[dev] + g_next_counter.fetch_add(1) % kCounterRing;
    CLPK_CUDA(cudaMemsetAsync(*out, 0, sizeof(unsigned long long), s));
    return CLPK_OK;
}

} // namespace clpk

using namespace clpk;

extern "C" {

int clpk_global_bandwidth(int width, const float *d_in, float *d_out, uint64_t n_floats, void *stream)
{
    int rc = require_sm100();
    if (rc != CLPK_OK)
        return rc;
    CLPK_REQUIRE(width == 1 || width == 2 || width == 4, "width must be 1, 2 or 4 (got %d)", width);
    CLPK_REQUIRE(d_in && d_out, "NULL buffer");
    const uint64_t per_block = 256ull * kFetchPerWI * (uint64_t)width;
    CLPK_REQUIRE(n_floats > 0 && n_floats % per_block == 0,
                 "n_floats (%llu) must be a positive multiple of %llu",
                 (unsigned long long)n_floats, (unsigned long long)per_block);
    const uint64_t blocks = n_floats / per_block;
    CLPK_REQUIRE(blocks <= 0x7FFFFFFFull, "too many blocks (%llu)", (unsigned long long)blocks);
    cudaStream_t s = as_stream(stream);
    if (width == 1)
        global_bandwidth_kernel<float><<<(unsigned)blocks, 256, 0, s>>>(d_in, d_out);
    else if (width == 2)
        global_bandwidth_kernel<float2>
            <<<(unsigned)blocks, 256, 0, s>>>(reinterpret_cast<const float2 *>(d_in), d_out);
    else
        global_bandwidth_kernel<float4>
            <<<(unsigned)blocks, 256, 0, s>>>(reinterpret_cast<const float4 *>(d_in), d_out);
    CLPK_LAUNCH_CHECK("global_bandwidth");
    return CLPK_OK;
}

int clpk_stream_read_grid(int variant, int *grid)
{
    int rc = require_sm100();
    if (rc != CLPK_OK)
        return rc;
    CLPK_REQUIRE(grid, "grid is NULL");
    CLPK_REQUIRE(known_variant(variant), "unknown variant %d", variant);
    *grid = read_grid(variant);
    return CLPK_OK;
}

int clpk_stream_read(int variant, const void *d_src, uint64_t n_bytes, uint32_t *d_partials, void *stream)
{
    int rc = require_sm100();
    if (rc != CLPK_OK)
        return rc;
    CLPK_REQUIRE(known_variant(variant), "unknown variant %d", variant);
    CLPK_REQUIRE(d_src && d_partials, "NULL buffer");
    CLPK_REQUIRE(n_bytes % 16 == 0 && ((uintptr_t)d_src % 16) == 0, "n_bytes and d_src must be 16-byte aligned");
    cudaStream_t s = as_stream(stream);
    const int grid = read_grid(variant);
    if (variant == CLPK_STREAM_WIDE) {
        CLPK_REQUIRE(((uintptr_t)d_src % 32) == 0, "the 256-bit variant needs a 32-byte aligned pointer");
        const uint64_t n_tiles = n_bytes / kWideTileBytes;
        CLPK_REQUIRE(n_tiles < 0x7FFFFFFFull, "n_bytes too large for one CTA per 8 KiB tile");
        CLPK_CUDA(cudaMemsetAsync(d_partials, 0, kWideSlots * sizeof(uint32_t), s));
        stream_read_wide<<<wide_grid(n_tiles), kWideThreads, 0, s>>>(reinterpret_cast<const Vec32 *>(d_src), n_tiles,
                                                                     (n_bytes % kWideTileBytes) / 16, d_partials);
    } else if (variant == CLPK_STREAM_LDG) {
        stream_read_ldg<<<grid, kLdgThreads, 0, s>>>(reinterpret_cast<const uint4 *>(d_src), n_bytes / 16,
                                                     d_partials);
    } else {
        uint32_t *st;
        rc = status_word(&st);
        if (rc != CLPK_OK)
            return rc;
        CLPK_CUDA(cudaFuncSetAttribute(stream_read_tma, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kTmaSmem));
        unsigned long long *ctr;
        rc = tile_counter(s, &ctr);
        if (rc != CLPK_OK)
            return rc;
        stream_read_tma<<<grid, 160, kTmaSmem, s>>>(reinterpret_cast<const uint8_t *>(d_src), n_bytes,
                                                    d_partials, st, ctr);
    }
    CLPK_LAUNCH_CHECK("stream_read");
    return CLPK_OK;
}

int clpk_stream_copy(int variant, void *d_dst, const void *d_src, uint64_t n_bytes, void *stream)
{
    int rc = require_sm100();
    if (rc != CLPK_OK)
        return rc;
    CLPK_REQUIRE(known_variant(variant), "unknown variant %d", variant);
    CLPK_REQUIRE(d_dst && d_src, "NULL buffer");
    CLPK_REQUIRE(n_bytes % 16 == 0 && ((uintptr_t)d_src % 16) == 0 && ((uintptr_t)d_dst % 16) == 0,
                 "n_bytes and both pointers must be 16-byte aligned");
    cudaStream_t s = as_stream(stream);
    if (variant == CLPK_STREAM_WIDE) {
        CLPK_REQUIRE(((uintptr_t)d_src % 32) == 0 && ((uintptr_t)d_dst % 32) == 0,
                     "the 256-bit variant needs 32-byte aligned pointers");
        const uint64_t n_tiles = n_bytes / kWideTileBytes;
        CLPK_REQUIRE(n_tiles < 0x7FFFFFFFull, "n_bytes too large for one CTA per 8 KiB tile");
        stream_copy_wide<<<wide_grid(n_tiles), kWideThreads, 0, s>>>(reinterpret_cast<Vec32 *>(d_dst),
                                                                     reinterpret_cast<const Vec32 *>(d_src), n_tiles,
                                                                     (n_bytes % kWideTileBytes) / 16);
    } else if (variant == CLPK_STREAM_LDG) {
        stream_copy_ldg<<<num_sms() * kLdgCtasPerSm, kLdgThreads, 0, s>>>(
            reinterpret_cast<uint4 *>(d_dst), reinterpret_cast<const uint4 *>(d_src), n_bytes / 16);
    } else {
        uint32_t *st;
        rc = status_word(&st);
        if (rc != CLPK_OK)
            return rc;
        CLPK_CUDA(cudaFuncSetAttribute(stream_copy_tma, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kTmaSmem));
        unsigned long long *ctr;
        rc = tile_counter(s, &ctr);
        if (rc != CLPK_OK)
            return rc;
        stream_copy_tma<<<num_sms(), 32, kTmaSmem, s>>>(reinterpret_cast<uint8_t *>(d_dst),
                                                        reinterpret_cast<const uint8_t *>(d_src), n_bytes, st, ctr);
    }
    CLPK_LAUNCH_CHECK("stream_copy");
    return CLPK_OK;
}

int clpk_stream_triad(int variant, float *d_a, const float *d_b, const float *d_c, float sc,
                      uint64_t n_floats, void *stream)
{
    int rc = require_sm100();
    if (rc != CLPK_OK)
        return rc;
    CLPK_REQUIRE(known_variant(variant), "unknown variant %d", variant);
    CLPK_REQUIRE(d_a && d_b && d_c, "NULL buffer");
    CLPK_REQUIRE(((uintptr_t)d_a % 16) == 0 && ((uintptr_t)d_b % 16) == 0 && ((uintptr_t)d_c % 16) == 0,
                 "pointers must be 16-byte aligned");
    cudaStream_t s = as_stream(stream);
    if (variant == CLPK_STREAM_WIDE) {
        CLPK_REQUIRE(((uintptr_t)d_a % 32) == 0 && ((uintptr_t)d_b % 32) == 0 && ((uintptr_t)d_c % 32) == 0,
                     "the 256-bit variant needs 32-byte aligned pointers");
        const uint64_t n_tiles = n_floats * 4 / kWideTileBytes;
        CLPK_REQUIRE(n_tiles < 0x7FFFFFFFull, "n_floats too large for one CTA per 8 KiB tile");
        stream_triad_wide<<<wide_grid(n_tiles), kWideThreads, 0, s>>>(
            reinterpret_cast<Vec32 *>(d_a), reinterpret_cast<const Vec32 *>(d_b), reinterpret_cast<const Vec32 *>(d_c), sc,
            n_tiles, n_floats - n_tiles * (kWideTileBytes / 4));
    } else if (variant == CLPK_STREAM_LDG) {
        stream_triad_ldg<<<num_sms() * kLdgCtasPerSm, kLdgThreads, 0, s>>>(
            reinterpret_cast<float4 *>(d_a), reinterpret_cast<const float4 *>(d_b),
            reinterpret_cast<const float4 *>(d_c), sc, n_floats / 4, n_floats % 4);
    } else {
        CLPK_REQUIRE(n_floats % 4 == 0, "the TMA variant needs n_floats to be a multiple of 4");
        uint32_t *st;
        rc = status_word(&st);
        if (rc != CLPK_OK)
            return rc;
        CLPK_CUDA(cudaFuncSetAttribute(stream_triad_tma, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kTmaTriadSmem));
        unsigned long long *ctr;
        rc = tile_counter(s, &ctr);
        if (rc != CLPK_OK)
            return rc;
        stream_triad_tma<<<num_sms(), 192, kTmaTriadSmem, s>>>(d_a, d_b, d_c, sc, n_floats * 4, st, ctr);
    }
    CLPK_LAUNCH_CHECK("stream_triad");
    return CLPK_OK;
}

/* Reads and clears the device-side status word of the TMA streaming kernels
 * (0 = no wait expired).  Synchronises the stream. */
int clpk_stream_status(uint32_t *h_status, void *stream)
{
    CLPK_REQUIRE(h_status, "h_status is NULL");
    uint32_t *st;
    int rc = status_word(&st);
    if (rc != CLPK_OK)
        return rc;
    CLPK_CUDA(cudaMemcpyAsync(h_status, st, sizeof(uint32_t), cudaMemcpyDeviceToHost, as_stream(stream)));
    CLPK_CUDA(cudaStreamSynchronize(as_stream(stream)));
    if (*h_status) {
        CLPK_CUDA(cudaMemsetAsync(st, 0, sizeof(uint32_t), as_stream(stream)));
        set_error("a TMA streaming kernel gave up waiting (code %u)", *h_status);
        return CLPK_ERR_TIMEOUT;
    }
    return CLPK_OK;
}

} // extern "C"
