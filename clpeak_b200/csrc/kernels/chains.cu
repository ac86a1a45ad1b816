// fp32 multiply-add chains, the pointer chase and the launch-latency probe.
#include <cuda.h>

#include <chrono>
#include <random>
#include <vector>

#include "../clpk_internal.h"
#include "../clpk_rng.h"

namespace clpk {

// ---- reference chain: x = fma(x, x, c), 128 x 16 dependent FMAs ------------------

#define CLPK_MAD_4(x, c)  x = __fmaf_rn(x, x, c); x = __fmaf_rn(x, x, c); x = __fmaf_rn(x, x, c); x = __fmaf_rn(x, x, c);
#define CLPK_MAD_16(x, c) CLPK_MAD_4(x, c) CLPK_MAD_4(x, c) CLPK_MAD_4(x, c) CLPK_MAD_4(x, c)

__global__ void __launch_bounds__(256) compute_sp_kernel(float *__restrict__ out, float a)
{
    float x = a;
    const float c = (float)threadIdx.x;
#pragma unroll
    for (int i = 0; i < 128; i++) {
        CLPK_MAD_16(x, c)
    }
    out[(uint64_t)blockIdx.x * 256 + threadIdx.x] = x;
}

// ---- seeded chain: x = fma(x, y, x) on a float4 per work-item ----------------------
// Four independent chains per thread; `iters` is a multiple of 16 and the body
// is unrolled 16 deep, so the loop overhead is 1/64 of the FMA count.

__global__ void __launch_bounds__(256) mad_chain_kernel(float *__restrict__ out, uint64_t seed,
                                                        float y, uint32_t iters)
{
    const uint64_t i = (uint64_t)blockIdx.x * 256 + threadIdx.x;
    float x0 = clpk_uniform_pm1(seed, 4 * i + 0);
    float x1 = clpk_uniform_pm1(seed, 4 * i + 1);
    float x2 = clpk_uniform_pm1(seed, 4 * i + 2);
    float x3 = clpk_uniform_pm1(seed, 4 * i + 3);
    for (uint32_t k = 0; k < iters; k += 16) {
#pragma unroll
        for (int u = 0; u < 16; u++) {
            x0 = __fmaf_rn(x0, y, x0);
            x1 = __fmaf_rn(x1, y, x1);
            x2 = __fmaf_rn(x2, y, x2);
            x3 = __fmaf_rn(x3, y, x3);
        }
    }
    out[i] = __fadd_rn(__fadd_rn(__fadd_rn(x0, x1), x2), x3);
}

// ---- pointer chase --------------------------------------------------------------------

__global__ void pointer_chase_kernel(const uint32_t *__restrict__ next, uint32_t start,
                                     uint64_t hops, uint32_t *__restrict__ result)
{
    uint32_t cur = start;
    uint32_t x = 0;
    uint64_t t0, t1;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    for (uint64_t h = 0; h < hops; h++) {
        // plain (coherent) load: every hop depends on the previous one
        asm volatile("ld.global.u32 %0, [%1];" : "=r"(cur) : "l"(next + cur) : "memory");
        x ^= cur;
    }
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
    const uint64_t dt = t1 - t0;
    result[0] = cur;
    result[1] = x;
    result[2] = (uint32_t)dt;
    result[3] = (uint32_t)(dt >> 32);
}

__global__ void noop_kernel() {}

} // namespace clpk

using namespace clpk;

extern "C" {

int clpk_compute_sp(float *d_out, float a, uint32_t grid, void *stream)
{
    int rc = require_sm100();
    if (rc != CLPK_OK)
        return rc;
    CLPK_REQUIRE(d_out && grid > 0, "bad arguments");
    compute_sp_kernel<<<grid, 256, 0, as_stream(stream)>>>(d_out, a);
    CLPK_LAUNCH_CHECK("compute_sp");
    return CLPK_OK;
}

int clpk_mad_chain(float *d_out, uint64_t n_items, uint64_t seed, float y, uint32_t iters,
                   void *stream)
{
    int rc = require_sm100();
    if (rc != CLPK_OK)
        return rc;
    CLPK_REQUIRE(d_out, "d_out is NULL");
    CLPK_REQUIRE(n_items > 0 && n_items % 256 == 0, "n_items must be a positive multiple of 256");
    CLPK_REQUIRE(iters % 16 == 0, "iters must be a multiple of 16");
    CLPK_REQUIRE(n_items / 256 <= 0x7FFFFFFFull, "n_items too large");
    mad_chain_kernel<<<(unsigned)(n_items / 256), 256, 0, as_stream(stream)>>>(d_out, seed, y, iters);
    CLPK_LAUNCH_CHECK("mad_chain");
    return CLPK_OK;
}

int clpk_pointer_chase(const uint32_t *d_next, uint32_t start, uint64_t hops, uint32_t *d_result,
                       void *stream)
{
    int rc = require_sm100();
    if (rc != CLPK_OK)
        return rc;
    CLPK_REQUIRE(d_next && d_result, "NULL buffer");
    pointer_chase_kernel<<<1, 1, 0, as_stream(stream)>>>(d_next, start, hops, d_result);
    CLPK_LAUNCH_CHECK("pointer_chase");
    return CLPK_OK;
}

// Sattolo's algorithm (one cycle through all n entries), the construction of
// chaseLatencyNs in the reference (src/cpu/latency.cpp:50-60) with one node per
// 4-byte entry and a seeded 64-bit generator instead of mt19937(0xC0FFEE).
int clpk_build_chase_cycle(uint32_t *h_next, uint64_t n, uint64_t seed)
{
    CLPK_REQUIRE(h_next, "h_next is NULL");
    CLPK_REQUIRE(n >= 2 && n <= 0xFFFFFFFFull, "n must be in [2, 2^32)");
    std::vector<uint32_t> order(n);
    for (uint64_t i = 0; i < n; i++)
        order[i] = (uint32_t)i;
    for (uint64_t i = n - 1; i > 0; i--) {
        const uint64_t j = clpk_rand64(seed, i) % i;     // j in [0, i)
        const uint32_t tmp = order[i];
        order[i] = order[j];
        order[j] = tmp;
    }
    for (uint64_t i = 0; i < n; i++)
        h_next[order[i]] = order[(i + 1) % n];
    return CLPK_OK;
}

int clpk_launch_noop(void *stream)
{
    noop_kernel<<<1, 1, 0, as_stream(stream)>>>();
    CLPK_LAUNCH_CHECK("noop");
    return CLPK_OK;
}

// The reference times cuLaunchKernel + cuStreamSynchronize (src/cuda/kernel_latency.cpp:44-63),
// i.e. the driver's own launch without the runtime's <<<>>> layer on top.  The same two
// driver entry points are looked up through the runtime here (nothing links libcuda); if the
// lookup fails the runtime launch is timed instead.
namespace {
typedef CUresult (*DrvLaunch)(CUfunction, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, CUstream,
                              void **, void **);
typedef CUresult (*DrvSync)(CUstream);

struct DriverLaunch {
    DrvLaunch launch = nullptr;
    DrvSync sync = nullptr;
    CUfunction fn = nullptr;
    bool ok = false;
};

DriverLaunch driver_launch_of_noop()
{
    DriverLaunch d;
    void *sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuLaunchKernel", &sym, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
        return d;
    d.launch = reinterpret_cast<DrvLaunch>(sym);
    if (cudaGetDriverEntryPoint("cuStreamSynchronize", &sym, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
        return d;
    d.sync = reinterpret_cast<DrvSync>(sym);
    cudaFunction_t f = nullptr;
    if (cudaGetFuncBySymbol(&f, reinterpret_cast<const void *>(clpk::noop_kernel)) != cudaSuccess) {
        (void)cudaGetLastError();
        return d;
    }
    d.fn = reinterpret_cast<CUfunction>(f);
    d.ok = d.launch && d.sync && d.fn;
    return d;
}
} // namespace

int clpk_launch_latency(uint32_t iters, uint32_t warmup, double *mean_us, void *stream)
{
    CLPK_REQUIRE(mean_us && iters > 0, "bad arguments");
    cudaStream_t s = as_stream(stream);
    const DriverLaunch drv = driver_launch_of_noop();
    void *no_args[1] = {nullptr};
    // returns 0 on success; the launch and the wait, exactly what is timed
    auto once = [&](const char **what, cudaError_t *rt) -> int {
        if (drv.ok) {
            const CUresult lr = drv.launch(drv.fn, 1, 1, 1, 1, 1, 1, 0, reinterpret_cast<CUstream>(s), no_args, nullptr);
            const CUresult sr = drv.sync(reinterpret_cast<CUstream>(s));
            if (lr != CUDA_SUCCESS || sr != CUDA_SUCCESS) {
                *what = lr != CUDA_SUCCESS ? "cuLaunchKernel" : "cuStreamSynchronize";
                *rt = cudaErrorUnknown;
                return 1;
            }
            return 0;
        }
        noop_kernel<<<1, 1, 0, s>>>();
        const cudaError_t le = cudaGetLastError();
        const cudaError_t se = cudaStreamSynchronize(s);
        if (le != cudaSuccess || se != cudaSuccess) {
            *what = le != cudaSuccess ? "launch noop" : "cudaStreamSynchronize";
            *rt = le != cudaSuccess ? le : se;
            return 1;
        }
        return 0;
    };
    const char *what = "";
    cudaError_t rt = cudaSuccess;
    for (uint32_t w = 0; w < warmup; w++)
        if (once(&what, &rt))
            return cuda_fail(rt, what);
    double total_ns = 0.0;
    for (uint32_t i = 0; i < iters; i++) {
        const auto t0 = std::chrono::steady_clock::now();
        const int bad = once(&what, &rt);
        const auto t1 = std::chrono::steady_clock::now();
        if (bad)
            return cuda_fail(rt, what);
        total_ns += (double)std::chrono::duration_cast<std::chrono::nanoseconds>(t1 - t0).count();
    }
    *mean_us = total_ns / 1000.0 / (double)iters;
    return CLPK_OK;
}

// The same empty kernel submitted `nodes` at a time as one CUDA graph: what a launch costs when
// a launch-bound loop is captured once and replayed (no reference counterpart: its latency test,
// src/cuda/kernel_latency.cpp:44-63, only has the one-kernel round trip).  mean_us_per_node =
// (graph launch + synchronise) / nodes, averaged over `iters` replays.
int clpk_graph_launch_latency(uint32_t nodes, uint32_t iters, uint32_t warmup, double *mean_us_per_node, void *stream)
{
    CLPK_REQUIRE(mean_us_per_node && iters > 0 && nodes > 0 && nodes <= 65536, "bad arguments");
    cudaStream_t own = nullptr, s = as_stream(stream);
    if (!s) {                                   // the legacy default stream cannot be captured
        CLPK_CUDA(cudaStreamCreateWithFlags(&own, cudaStreamNonBlocking));
        s = own;
    }
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    auto cleanup = [&] {
        if (exec)
            cudaGraphExecDestroy(exec);
        if (graph)
            cudaGraphDestroy(graph);
        if (own)
            cudaStreamDestroy(own);
    };
    cudaError_t e = cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal);
    if (e != cudaSuccess) {
        cleanup();
        return cuda_fail(e, "cudaStreamBeginCapture");
    }
    for (uint32_t i = 0; i < nodes; i++)
        noop_kernel<<<1, 1, 0, s>>>();
    e = cudaStreamEndCapture(s, &graph);
    if (e == cudaSuccess)
        e = cudaGraphInstantiate(&exec, graph, 0);
    if (e != cudaSuccess) {
        cleanup();
        return cuda_fail(e, "graph capture / instantiate");
    }
    double total_ns = 0.0;
    for (uint32_t i = 0; i < warmup + iters; i++) {
        const auto t0 = std::chrono::steady_clock::now();
        e = cudaGraphLaunch(exec, s);
        if (e == cudaSuccess)
            e = cudaStreamSynchronize(s);
        const auto t1 = std::chrono::steady_clock::now();
        if (e != cudaSuccess) {
            cleanup();
            return cuda_fail(e, "cudaGraphLaunch");
        }
        if (i >= warmup)
            total_ns += (double)std::chrono::duration_cast<std::chrono::nanoseconds>(t1 - t0).count();
    }
    cleanup();
    *mean_us_per_node = total_ns / 1000.0 / (double)iters / (double)nodes;
    return CLPK_OK;
}

} // extern "C"
