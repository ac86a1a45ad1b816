// A streaming-read checksum that allocates nothing.
//
// clpk_stream_read() hands its per-CTA partial XORs back in a buffer the caller
// allocates.  Some callers cannot allocate device memory at the moment they
// need the checksum: code on a latency-critical path where cudaMalloc's implicit
// device synchronisation is not acceptable, a plugin whose host forbids
// allocator calls after start-up, or a process running with its memory pool
// already handed out in full.  For them this entry point keeps the partials in
// a fixed array that lives in the library's own device image.  The first call
// on a device looks the array's device address up (cudaGetSymbolAddress); make
// that first call before any stream capture.
//
// The array (kMaxCtas partial words plus a ticket counter, 16.25 KiB) exists
// once per GPU that loads the library and stays until the process exits.  Every
// call on a device shares it, so calls that overlap on the GPU -- two streams,
// two host threads -- race on it and must be serialised by the caller.  The
// array keeps the last call's partials; the only word that has to start at zero,
// the ticket, is cleared by a memset at the head of every call.
#include <atomic>

#include "../clpk_internal.h"

namespace clpk {

constexpr uint32_t kMaxCtas = 4096;                  // capacity of the static scratch
constexpr uint32_t kTicket = kMaxCtas;               // index of the arrival counter
constexpr int kThreads = 512;
constexpr int kUnroll = 4;

// File-scope scratch.  In host code this name is only a stand-in for the symbol;
// the usable device address comes from cudaGetSymbolAddress (scratch_for_device).
static __device__ __align__(256) uint32_t g_read_scratch[kMaxCtas + 64];

__device__ __forceinline__ uint32_t xor_uint4(const uint4 &v) { return v.x ^ v.y ^ v.z ^ v.w; }

__global__ void __launch_bounds__(kThreads) stream_checksum_static(const uint4 *__restrict__ src, uint64_t n16,
                                                                   uint32_t *__restrict__ scratch,
                                                                   uint32_t *__restrict__ out)
{
    constexpr uint64_t kTile = (uint64_t)kThreads * kUnroll;
    uint32_t acc = 0;
    const uint64_t n_full = n16 / kTile;
    for (uint64_t t = blockIdx.x; t < n_full; t += gridDim.x) {
        const uint4 *p = src + t * kTile + threadIdx.x;
        uint4 v[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; u++)
            v[u] = __ldcs(p + u * kThreads);
#pragma unroll
        for (int u = 0; u < kUnroll; u++)
            acc ^= xor_uint4(v[u]);
    }
    if (blockIdx.x == 0)
        for (uint64_t i = n_full * kTile + threadIdx.x; i < n16; i += kThreads)
            acc ^= xor_uint4(__ldcs(src + i));

    __shared__ uint32_t warp_x[kThreads / 32];
    __shared__ bool is_last;
    for (int o = 16; o > 0; o >>= 1)
        acc ^= __shfl_xor_sync(0xffffffffu, acc, o);
    if ((threadIdx.x & 31) == 0)
        warp_x[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        uint32_t x = 0;
        for (int w = 0; w < kThreads / 32; w++)
            x ^= warp_x[w];
        scratch[blockIdx.x] = x;
        __threadfence();                                       // partial visible before the ticket
        is_last = atomicAdd(&scratch[kTicket], 1u) == gridDim.x - 1;
    }
    __syncthreads();
    if (!is_last)
        return;
    // The last CTA to arrive folds every partial.
    __threadfence();
    uint32_t x = 0;
    for (uint32_t i = threadIdx.x; i < gridDim.x; i += kThreads)
        x ^= __ldcg(scratch + i);
    for (int o = 16; o > 0; o >>= 1)
        x ^= __shfl_xor_sync(0xffffffffu, x, o);
    if ((threadIdx.x & 31) == 0)
        warp_x[threadIdx.x >> 5] = x;
    __syncthreads();
    if (threadIdx.x == 0) {
        uint32_t y = 0;
        for (int w = 0; w < kThreads / 32; w++)
            y ^= warp_x[w];
        *out = y;
    }
}

// Device address of the scratch array on the current device, resolved with that
// device current.  Two host threads making their first call on one device at the
// same moment both resolve it and both store the same value; the slots are atomic
// so that this is not a data race.
static std::atomic<uint32_t *> g_scratch_ptr[64];

static int scratch_for_device(uint32_t **out)
{
    int dev = 0;
    CLPK_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) {
        set_error("device index %d out of range", dev);
        return CLPK_ERR_BAD_ARG;
    }
    uint32_t *ptr = g_scratch_ptr[dev].load(std::memory_order_acquire);
    if (!ptr) {
        CLPK_CUDA(cudaGetSymbolAddress((void **)&ptr, g_read_scratch));
        g_scratch_ptr[dev].store(ptr, std::memory_order_release);
    }
    *out = ptr;
    return CLPK_OK;
}

} // namespace clpk

using namespace clpk;

extern "C" int clpk_stream_checksum_static(const void *d_src, uint64_t n_bytes, uint32_t grid_ctas,
                                           uint32_t *d_xor_out, void *stream)
{
    int rc = require_sm100();
    if (rc != CLPK_OK)
        return rc;
    CLPK_REQUIRE(d_src && d_xor_out, "NULL buffer");
    CLPK_REQUIRE(n_bytes % 16 == 0 && ((uintptr_t)d_src % 16) == 0, "n_bytes and d_src must be 16-byte aligned");
    const uint32_t grid = grid_ctas ? grid_ctas : (uint32_t)num_sms() * 4u;
    if (grid > kMaxCtas) {
        set_error("clpk_stream_checksum_static: %u CTAs requested, the static scratch holds partials for at most %u",
                  grid, kMaxCtas);
        return CLPK_ERR_TOO_LARGE;
    }
    uint32_t *scratch = nullptr;
    rc = scratch_for_device(&scratch);
    if (rc != CLPK_OK)
        return rc;
    cudaStream_t s = as_stream(stream);
    CLPK_CUDA(cudaMemsetAsync(scratch + kTicket, 0, sizeof(uint32_t), s));
    stream_checksum_static<<<grid, kThreads, 0, s>>>(static_cast<const uint4 *>(d_src), n_bytes / 16, scratch,
                                                     d_xor_out);
    CLPK_LAUNCH_CHECK("stream_checksum_static");
    return CLPK_OK;
}
