// Device, memory, stream and event plumbing behind the C ABI.
#include <stdarg.h>
#include <stdlib.h>
#include <string.h>

#include <atomic>
#include <mutex>

#include "../clpk_internal.h"

namespace clpk {

static thread_local char g_err[512] = "";

void set_error(const char *fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

int cuda_fail(cudaError_t e, const char *what)
{
    set_error("%s: %s (%s)", what, cudaGetErrorString(e), cudaGetErrorName(e));
    // The runtime also keeps a failed call's code as its "last error"; this failure is reported here, so take it
    // back out, or the next kernel launch's check would report it a second time (a sticky error stays whatever we do).
    (void)cudaGetLastError();
    if (e == cudaErrorNoDevice || e == cudaErrorInsufficientDriver ||
        e == cudaErrorInitializationError)
        return CLPK_ERR_NO_DEVICE;
    return CLPK_ERR_CUDA;
}

struct DevCache {
    bool valid = false;
    int major = 0, minor = 0, sms = 0, smem_optin = 0;
};
static DevCache g_dev[64];

static int load_cache(int *dev_out)
{
    int dev = 0;
    CLPK_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) {
        set_error("device index %d out of range", dev);
        return CLPK_ERR_BAD_ARG;
    }
    DevCache &c = g_dev[dev];
    if (!c.valid) {
        CLPK_CUDA(cudaDeviceGetAttribute(&c.major, cudaDevAttrComputeCapabilityMajor, dev));
        CLPK_CUDA(cudaDeviceGetAttribute(&c.minor, cudaDevAttrComputeCapabilityMinor, dev));
        CLPK_CUDA(cudaDeviceGetAttribute(&c.sms, cudaDevAttrMultiProcessorCount, dev));
        CLPK_CUDA(cudaDeviceGetAttribute(&c.smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
        c.valid = true;
    }
    *dev_out = dev;
    return CLPK_OK;
}

int require_sm100()
{
    int dev = 0;
    int rc = load_cache(&dev);
    if (rc != CLPK_OK)
        return rc;
    if (g_dev[dev].major != 10) {
        set_error("device %d is sm_%d%d; these kernels are built for sm_100a only", dev,
                  g_dev[dev].major, g_dev[dev].minor);
        return CLPK_ERR_UNSUPPORTED;
    }
    return CLPK_OK;
}

int num_sms()
{
    int dev = 0;
    if (load_cache(&dev) != CLPK_OK)
        return 0;
    return g_dev[dev].sms;
}

int smem_optin_bytes()
{
    int dev = 0;
    if (load_cache(&dev) != CLPK_OK)
        return 0;
    return g_dev[dev].smem_optin;
}

static std::atomic<int> g_tune[CLPK_TUNE_COUNT];
static std::once_flag g_tune_once;

static void load_tuning_from_environment()
{
    static const char *names[CLPK_TUNE_COUNT] = {"CLPK_GEMM_NO_ALIGN", "CLPK_GEMM_ALIGN_AT", "CLPK_GEMM_GROUP",
                                                 "CLPK_MMA_PAIR", "CLPK_GEMM_FP4_TILE", "CLPK_MMA_LONE_LANE", "CLPK_GEMM_NO_PDL"};
    for (int k = 0; k < CLPK_TUNE_COUNT; k++) {
        const char *e = getenv(names[k]);
        g_tune[k].store((e && e[0]) ? atoi(e) : -1);
    }
}

int tuning(int knob)
{
    std::call_once(g_tune_once, load_tuning_from_environment);
    return (knob >= 0 && knob < CLPK_TUNE_COUNT) ? g_tune[knob].load(std::memory_order_relaxed) : -1;
}

} // namespace clpk

using namespace clpk;

extern "C" {

int clpk_set_tuning(int knob, int value)
{
    CLPK_REQUIRE(knob >= 0 && knob < CLPK_TUNE_COUNT, "unknown tuning knob %d", knob);
    (void)tuning(knob);                    // the environment is read first, so that it cannot overwrite this later
    g_tune[knob].store(value < 0 ? -1 : value);
    return CLPK_OK;
}

int clpk_get_tuning(int knob, int *value)
{
    CLPK_REQUIRE(knob >= 0 && knob < CLPK_TUNE_COUNT && value, "unknown tuning knob %d or NULL value", knob);
    *value = tuning(knob);
    return CLPK_OK;
}

const char *clpk_last_error(void) { return g_err; }
const char *clpk_version(void) { return "clpeak-b200 0.1 (sm_100a)"; }

int clpk_device_count(int *count)
{
    CLPK_REQUIRE(count, "count is NULL");
    *count = 0;
    cudaError_t e = cudaGetDeviceCount(count);
    if (e != cudaSuccess) {
        *count = 0;
        return cuda_fail(e, "cudaGetDeviceCount");
    }
    return CLPK_OK;
}

int clpk_device_info(int device, clpk_device_info_t *out)
{
    CLPK_REQUIRE(out, "out is NULL");
    memset(out, 0, sizeof(*out));
    cudaDeviceProp p;
    CLPK_CUDA(cudaGetDeviceProperties(&p, device));
    strncpy(out->name, p.name, sizeof(out->name) - 1);
    out->cc_major = p.major;
    out->cc_minor = p.minor;
    out->num_sms = p.multiProcessorCount;
    out->total_mem_bytes = p.totalGlobalMem;
    CLPK_CUDA(cudaDriverGetVersion(&out->driver_version));
    CLPK_CUDA(cudaRuntimeGetVersion(&out->runtime_version));
    CLPK_CUDA(cudaDeviceGetAttribute(&out->sm_clock_khz, cudaDevAttrClockRate, device));
    CLPK_CUDA(cudaDeviceGetAttribute(&out->mem_clock_khz, cudaDevAttrMemoryClockRate, device));
    out->mem_bus_bits = p.memoryBusWidth;
    out->l2_bytes = p.l2CacheSize;
    out->smem_optin_bytes = (int)p.sharedMemPerBlockOptin;
    return CLPK_OK;
}

int clpk_set_device(int device)
{
    CLPK_CUDA(cudaSetDevice(device));
    return CLPK_OK;
}

int clpk_malloc(void **d_ptr, size_t bytes)
{
    CLPK_REQUIRE(d_ptr, "d_ptr is NULL");
    *d_ptr = nullptr;
    CLPK_CUDA(cudaMalloc(d_ptr, bytes ? bytes : 1));
    return CLPK_OK;
}

int clpk_free(void *d_ptr)
{
    if (d_ptr)
        CLPK_CUDA(cudaFree(d_ptr));
    return CLPK_OK;
}

int clpk_malloc_host(void **h_ptr, size_t bytes)
{
    CLPK_REQUIRE(h_ptr, "h_ptr is NULL");
    *h_ptr = nullptr;
    CLPK_CUDA(cudaMallocHost(h_ptr, bytes ? bytes : 1));
    return CLPK_OK;
}

int clpk_free_host(void *h_ptr)
{
    if (h_ptr)
        CLPK_CUDA(cudaFreeHost(h_ptr));
    return CLPK_OK;
}

int clpk_memset(void *d_ptr, int byte, size_t bytes, void *stream)
{
    CLPK_CUDA(cudaMemsetAsync(d_ptr, byte, bytes, as_stream(stream)));
    return CLPK_OK;
}

int clpk_memcpy_h2d(void *d_dst, const void *h_src, size_t bytes, void *stream)
{
    CLPK_CUDA(cudaMemcpyAsync(d_dst, h_src, bytes, cudaMemcpyHostToDevice, as_stream(stream)));
    return CLPK_OK;
}

int clpk_memcpy_d2h(void *h_dst, const void *d_src, size_t bytes, void *stream)
{
    CLPK_CUDA(cudaMemcpyAsync(h_dst, d_src, bytes, cudaMemcpyDeviceToHost, as_stream(stream)));
    return CLPK_OK;
}

int clpk_memcpy_d2d(void *d_dst, const void *d_src, size_t bytes, void *stream)
{
    CLPK_CUDA(cudaMemcpyAsync(d_dst, d_src, bytes, cudaMemcpyDeviceToDevice, as_stream(stream)));
    return CLPK_OK;
}

int clpk_stream_create(void **stream)
{
    CLPK_REQUIRE(stream, "stream is NULL");
    cudaStream_t s;
    CLPK_CUDA(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
    *stream = s;
    return CLPK_OK;
}

int clpk_stream_destroy(void *stream)
{
    if (stream)
        CLPK_CUDA(cudaStreamDestroy(as_stream(stream)));
    return CLPK_OK;
}

int clpk_stream_sync(void *stream)
{
    CLPK_CUDA(cudaStreamSynchronize(as_stream(stream)));
    return CLPK_OK;
}

int clpk_event_create(void **event)
{
    CLPK_REQUIRE(event, "event is NULL");
    cudaEvent_t e;
    CLPK_CUDA(cudaEventCreate(&e));
    *event = e;
    return CLPK_OK;
}

int clpk_event_destroy(void *event)
{
    if (event)
        CLPK_CUDA(cudaEventDestroy(reinterpret_cast<cudaEvent_t>(event)));
    return CLPK_OK;
}

int clpk_event_record(void *event, void *stream)
{
    CLPK_CUDA(cudaEventRecord(reinterpret_cast<cudaEvent_t>(event), as_stream(stream)));
    return CLPK_OK;
}

int clpk_event_sync(void *event)
{
    CLPK_CUDA(cudaEventSynchronize(reinterpret_cast<cudaEvent_t>(event)));
    return CLPK_OK;
}

int clpk_event_elapsed_ms(void *start, void *stop, float *ms)
{
    CLPK_REQUIRE(ms, "ms is NULL");
    CLPK_CUDA(cudaEventElapsedTime(ms, reinterpret_cast<cudaEvent_t>(start),
                                   reinterpret_cast<cudaEvent_t>(stop)));
    return CLPK_OK;
}

} // extern "C"
