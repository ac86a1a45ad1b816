// Launcher for the reference project's OWN CUDA kernels, for measuring what they
// reach on the GPU this backend is written for.  Test/bench infrastructure only: the
// product never loads it.
//
// The kernels are not in this repository.  `make refcuda` compiles each
// src/cuda/cuda_kernels/<name>.cu of the reference checkout, where it lies, into
// <dir>/<name>.cubin; this program loads those cubins through the CUDA driver API and
// launches them with the geometry, launch count calibration and accounting of the
// reference's host side:
//   grid / block / bytes per block, value = threads * work / time
//                                  src/cuda/compute_kernel.cpp:49-92
//   warm-up, one-launch probe, batch sized to the time budget
//                                  src/cuda/cuda_peak.cpp:64-107, src/common/common.cpp:35-45
//   targetGlobalThreads            include/common/common.h:142-147
//   per-row descriptors            src/cuda/compute_float.cpp:10-125, src/cuda/compute_int.cpp:10-64,
//                                  src/cuda/wmma.cpp:20-420
//   global / local / image / latency rows
//                                  src/cuda/global_bandwidth.cpp:6-92, src/cuda/local_bandwidth.cpp:15-60,
//                                  src/cuda/image_bandwidth.cpp:20-107, src/cuda/kernel_latency.cpp:6-80
// Rows the reference itself skips on this architecture (the sm_120a-only fp4 block-scale
// `mma.sync` forms, int4) are reported as skipped; their kernels do not assemble for sm_100a.
//
// usage: ref_cuda_runner <cubin dir> [--budget-us N (default 500000)] [--filter substring] [--csv file]
//        ref_cuda_runner <cubin dir> --dump <test>/<label> <out file> [--blocks N] [--arg X]
//                                    [--input file] [--dim W H]
// The second form is the parity pin: it launches ONE reference kernel once on a small grid and
// writes the bytes of its output buffer to <out file>, so that a test can compare the
// reference's own result with the CPU oracle and with this backend's kernel on the same
// inputs.  Rows: the shader-core chains (single_precision_compute/float ...
// integer_compute_int8_dp/int8_dp8; --arg replaces the scalar the reference's host passes),
// global_memory_bandwidth/{float,float2,float4} (--input: raw fp32, blocks*256*16*width values),
// local_memory_bandwidth/{float,float2,float4}, image_memory_bandwidth/float4 (--dim W H,
// --input: W*H*4 raw fp32; the grid is W*H/16/256 blocks as in src/cuda/image_bandwidth.cpp:20-107).
// The first form prints one JSON object per row on stdout.  --csv also writes the rows as a result file of the
// reference's CSV schema (format_version 2; writer src/common/result_store.cpp:264), with the
// reference's test tags and metric labels, so that `clpeak --cuda --compare <file>` lines the
// two backends up row by row.
#include <cuda.h>

#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

namespace {

#define DRV(call)                                                                      \
    do {                                                                               \
        CUresult rc_ = (call);                                                         \
        if (rc_ != CUDA_SUCCESS) {                                                     \
            const char *name_ = nullptr;                                               \
            cuGetErrorName(rc_, &name_);                                               \
            std::fprintf(stderr, "%s:%d: %s -> %s\n", __FILE__, __LINE__, #call,       \
                         name_ ? name_ : "?");                                         \
            std::exit(3);                                                              \
        }                                                                              \
    } while (0)

struct Gpu {
    CUdevice dev = 0;
    CUcontext ctx = nullptr;
    CUstream stream = nullptr;
    int sms = 0;
    size_t vram = 0;
    std::string dir;
    unsigned budget_us = 500000;
};

constexpr unsigned kWarmups = 2;          // options.h:40
constexpr unsigned kMaxLaunches = 100000; // cap on one timed batch

uint64_t target_threads(int sms)
{
    const uint64_t floor_threads = 32ull << 20, scaled = (uint64_t)sms * 2048ull * 256ull;
    return scaled > floor_threads ? scaled : floor_threads;
}

bool load_kernel(const Gpu &g, const char *module, const char *kernel, CUmodule *mod, CUfunction *fn)
{
    const std::string path = g.dir + "/" + module + ".cubin";
    if (cuModuleLoad(mod, path.c_str()) != CUDA_SUCCESS)
        return false;
    if (cuModuleGetFunction(fn, *mod, kernel) != CUDA_SUCCESS) {
        cuModuleUnload(*mod);
        return false;
    }
    return true;
}

// microseconds per launch: warm-ups each waited for, one timed launch to size the
// batch, then the batch between two events
double time_kernel(const Gpu &g, CUfunction fn, unsigned grid, unsigned block, void **args)
{
    CUevent t0, t1;
    DRV(cuEventCreate(&t0, CU_EVENT_DEFAULT));
    DRV(cuEventCreate(&t1, CU_EVENT_DEFAULT));
    auto batch = [&](unsigned n) {
        DRV(cuEventRecord(t0, g.stream));
        for (unsigned i = 0; i < n; i++)
            DRV(cuLaunchKernel(fn, grid, 1, 1, block, 1, 1, 0, g.stream, args, nullptr));
        DRV(cuEventRecord(t1, g.stream));
        DRV(cuEventSynchronize(t1));
        float ms = 0;
        DRV(cuEventElapsedTime(&ms, t0, t1));
        return (double)ms * 1000.0;
    };
    for (unsigned w = 0; w < kWarmups; w++) {
        DRV(cuLaunchKernel(fn, grid, 1, 1, block, 1, 1, 0, g.stream, args, nullptr));
        DRV(cuStreamSynchronize(g.stream));
    }
    double one = batch(1);
    if (one < 1.0)
        one = 1.0;
    double want = (double)g.budget_us / one;
    if (want < 1.0)
        want = 1.0;
    if (want > (double)kMaxLaunches)
        want = (double)kMaxLaunches;
    const unsigned n = (unsigned)want;
    const double total = batch(n);
    cuEventDestroy(t0);
    cuEventDestroy(t1);
    return total / n;
}

struct CsvRow {
    std::string test, label, unit, reason;
    double value;
    bool ok;
};
std::vector<CsvRow> g_rows;

void emit(const char *test, const char *label, const char *unit, double value, double us, unsigned grid)
{
    g_rows.push_back({test, label, unit, "", value, true});
    std::printf("{\"test\": \"%s\", \"label\": \"%s\", \"unit\": \"%s\", \"value\": %.6g, \"us_per_launch\": %.4f, "
                "\"grid\": %u}\n",
                test, label, unit, value, us, grid);
    std::fflush(stdout);
}

void emit_skip(const char *test, const char *label, const char *why, const char *unit = "")
{
    g_rows.push_back({test, label, unit, why, 0.0, false});
    std::printf("{\"test\": \"%s\", \"label\": \"%s\", \"skipped\": \"%s\"}\n", test, label, why);
    std::fflush(stdout);
}

enum class Arg { F32, F64, I32 };

struct ComputeRow {
    const char *test, *label, *module, *kernel, *unit;
    double divider;        // 1e9 for gflops/gops, 1e12 for tflops/tops
    unsigned block;        // threads per block
    unsigned out_per_block;
    unsigned elem_bytes;
    double work_per_thread;
    Arg arg_kind;
    double arg;
    const char *skip;      // non-null: the reference's own rule skips the row on sm_100
};

constexpr double kFp = 4096, kDot = 8192, kMma = 65536;
constexpr const char *kNeeds120 = "mma.sync with fp4 / block scale exists on sm_120a only";

const ComputeRow kComputeRows[] = {
    {"single_precision_compute", "float", "compute_sp", "compute_sp", "gflops", 1e9, 256, 256, 4, kFp, Arg::F32, 1.3, nullptr},
    {"half_precision_compute", "half", "compute_hp", "compute_hp", "gflops", 1e9, 256, 256, 4, kFp, Arg::F32, 1.3, nullptr},
    {"half_precision_compute", "half2", "compute_hp", "compute_hp2", "gflops", 1e9, 256, 256, 4, kFp, Arg::F32, 1.3, nullptr},
    {"double_precision_compute", "double", "compute_dp", "compute_dp", "gflops", 1e9, 256, 256, 8, kFp, Arg::F64, 1.3, nullptr},
    {"mixed_precision_compute", "mp", "compute_mp", "compute_mp", "gflops", 1e9, 256, 256, 4, kFp, Arg::F32, 1.3, nullptr},
    {"bfloat16_compute", "bf16", "compute_bf16", "compute_bf16", "gflops", 1e9, 256, 256, 4, kFp, Arg::F32, 1.3, nullptr},
    {"integer_compute", "int", "compute_int32", "compute_int32", "gops", 1e9, 256, 256, 4, kFp, Arg::I32, 3, nullptr},
    {"integer_compute_int8_dp", "int8_dp", "compute_int8_dp", "compute_int8_dp", "gops", 1e9, 256, 256, 4, kDot, Arg::I32, 4, nullptr},
    {"integer_compute_int8_dp", "int8_dp2", "compute_int8_dp", "compute_int8_dp2", "gops", 1e9, 256, 256, 4, kDot, Arg::I32, 4, nullptr},
    {"integer_compute_int8_dp", "int8_dp4", "compute_int8_dp", "compute_int8_dp4", "gops", 1e9, 256, 256, 4, kDot, Arg::I32, 4, nullptr},
    {"integer_compute_int8_dp", "int8_dp8", "compute_int8_dp", "compute_int8_dp8", "gops", 1e9, 256, 256, 4, kDot, Arg::I32, 4, nullptr},
    {"wmma_fp16", "wmma_fp16", "wmma_fp16", "wmma_fp16", "tflops", 1e12, 32, 256, 4, kMma * 4, Arg::F32, 1.3, nullptr},
    {"wmma_fp16_f16", "fp16_f16acc", "wmma_fp16_f16", "wmma_fp16_f16", "tflops", 1e12, 32, 32, 4, kMma * 4, Arg::F32, 1.3, nullptr},
    {"wmma_bf16", "wmma_bf16", "wmma_bf16", "wmma_bf16", "tflops", 1e12, 32, 256, 4, kMma * 4, Arg::F32, 1.3, nullptr},
    {"wmma_tf32", "wmma_tf32", "wmma_tf32", "wmma_tf32", "tflops", 1e12, 32, 128, 4, kMma * 2, Arg::F32, 1.3, nullptr},
    {"wmma_fp64", "wmma_fp64", "wmma_fp64", "wmma_fp64", "tflops", 1e12, 32, 64, 8, kMma, Arg::F64, 1.3, nullptr},
    {"wmma_fp8_e4m3", "fp8_e4m3", "wmma_fp8_e4m3", "wmma_fp8_e4m3", "tflops", 1e12, 32, 128, 4, kMma * 8, Arg::F32, 1.3, nullptr},
    {"wmma_fp8_e5m2", "fp8_e5m2", "wmma_fp8_e5m2", "wmma_fp8_e5m2", "tflops", 1e12, 32, 128, 4, kMma * 8, Arg::F32, 1.3, nullptr},
    {"wmma_fp4_e2m1", "fp4_e2m1", "", "", "tflops", 1e12, 32, 128, 4, kMma * 8, Arg::F32, 1.3, kNeeds120},
    {"wmma_mxf4_e2m1", "mxf4_e2m1", "", "", "tflops", 1e12, 32, 128, 4, kMma * 16, Arg::F32, 1.3, kNeeds120},
    {"wmma_nvf4_e2m1", "nvf4_e2m1", "", "", "tflops", 1e12, 32, 128, 4, kMma * 16, Arg::F32, 1.3, kNeeds120},
    {"wmma_mxf4_sparse", "mxf4_sparse", "", "", "tflops", 1e12, 32, 128, 4, kMma * 32, Arg::F32, 1.3, kNeeds120},
    {"wmma_nvf4_sparse", "nvf4_sparse", "", "", "tflops", 1e12, 32, 128, 4, kMma * 32, Arg::F32, 1.3, kNeeds120},
    {"wmma_int8", "wmma_int8", "wmma_int8", "wmma_int8", "tops", 1e12, 32, 256, 4, kMma * 4, Arg::I32, 3, nullptr},
    {"wmma_int8_k32", "int8_k32", "wmma_int8_k32", "wmma_int8_k32", "tops", 1e12, 32, 128, 4, kMma * 4, Arg::I32, 3, nullptr},
    {"wmma_int8_sparse", "int8_sparse", "wmma_int8_sparse", "wmma_int8_sparse", "tops", 1e12, 32, 128, 4, kMma * 4, Arg::I32, 3, nullptr},
    {"wmma_int4", "int4", "", "", "tops", 1e12, 32, 64, 4, kMma * 2, Arg::I32, 3,
     "int4 mma.sync is sm_75..sm_89 only"},
};

bool wanted(const char *filter, const char *test, const char *label)
{
    return !filter || std::strstr(test, filter) || std::strstr(label, filter);
}

void run_compute(const Gpu &g, const ComputeRow &r)
{
    if (r.skip) {
        emit_skip(r.test, r.label, r.skip, r.unit);
        return;
    }
    const uint64_t bytes_per_block = (uint64_t)r.out_per_block * r.elem_bytes;
    const uint64_t max_blocks = g.vram / 4 / bytes_per_block;
    uint64_t blocks = target_threads(g.sms) / r.block;
    if (blocks > max_blocks)
        blocks = max_blocks;
    const unsigned grid = (unsigned)blocks;
    CUmodule mod;
    CUfunction fn;
    if (!load_kernel(g, r.module, r.kernel, &mod, &fn)) {
        emit_skip(r.test, r.label, "cubin or kernel missing");
        return;
    }
    CUdeviceptr out = 0;
    DRV(cuMemAlloc(&out, (size_t)grid * bytes_per_block));
    float af = (float)r.arg;
    double ad = r.arg;
    int ai = (int)r.arg;
    void *scalar = r.arg_kind == Arg::F32 ? (void *)&af : r.arg_kind == Arg::F64 ? (void *)&ad : (void *)&ai;
    void *args[2] = {&out, scalar};
    const double us = time_kernel(g, fn, grid, r.block, args);
    const double threads = (double)grid * r.block;
    emit(r.test, r.label, r.unit, threads * r.work_per_thread * 1e6 / us / r.divider, us, grid);
    cuMemFree(out);
    cuModuleUnload(mod);
}

// any non-constant data will do: the fill only has to defeat memory compression
void fill_host(float *p, size_t n)
{
    uint32_t s = 0x2545F491u;
    for (size_t i = 0; i < n; i++) {
        s = s * 1664525u + 1013904223u;
        p[i] = (float)(s >> 8) * (1.0f / 16777216.0f);
    }
}

void run_global_bandwidth(const Gpu &g, const char *filter)
{
    const char *test = "global_memory_bandwidth";
    constexpr unsigned kBlock = 256, kFetch = 16;
    const uint64_t cap_bytes = 1ull << 29; // the GPU default of the reference's per-device config
    uint64_t items = g.vram / sizeof(float) / 4;
    if (items > cap_bytes / sizeof(float))
        items = cap_bytes / sizeof(float);
    items = items / (kBlock * kFetch) * (kBlock * kFetch);
    CUdeviceptr in = 0, out = 0;
    DRV(cuMemAlloc(&in, items * sizeof(float)));
    DRV(cuMemAlloc(&out, items * sizeof(float)));
    {
        std::vector<float> host(items);
        fill_host(host.data(), items);
        DRV(cuMemcpyHtoD(in, host.data(), items * sizeof(float)));
    }
    const struct { const char *label, *kernel; unsigned width; } variants[] = {
        {"float", "global_bandwidth_v1", 1}, {"float2", "global_bandwidth_v2", 2}, {"float4", "global_bandwidth_v4", 4}};
    for (const auto &v : variants) {
        if (!wanted(filter, test, v.label))
            continue;
        CUmodule mod;
        CUfunction fn;
        if (!load_kernel(g, "global_bandwidth", v.kernel, &mod, &fn)) {
            emit_skip(test, v.label, "cubin or kernel missing");
            continue;
        }
        uint64_t blocks = items / kFetch / v.width / kBlock;
        if (blocks == 0)
            blocks = 1;
        void *args[2] = {&in, &out};
        const double us = time_kernel(g, fn, (unsigned)blocks, kBlock, args);
        const double bytes = (double)blocks * kBlock * kFetch * v.width * sizeof(float);
        emit(test, v.label, "gbps", bytes / us / 1e3, us, (unsigned)blocks);
        cuModuleUnload(mod);
    }
    cuMemFree(in);
    cuMemFree(out);
}

void run_local_bandwidth(const Gpu &g, const char *filter)
{
    const char *test = "local_memory_bandwidth";
    const uint64_t threads = target_threads(g.sms);
    const unsigned grid = (unsigned)(threads / 256);
    CUdeviceptr out = 0;
    DRV(cuMemAlloc(&out, threads * sizeof(float)));
    const struct { const char *label, *kernel; unsigned width; } variants[] = {
        {"float", "local_bandwidth_v1", 1}, {"float2", "local_bandwidth_v2", 2}, {"float4", "local_bandwidth_v4", 4}};
    for (const auto &v : variants) {
        if (!wanted(filter, test, v.label))
            continue;
        CUmodule mod;
        CUfunction fn;
        if (!load_kernel(g, "local_bandwidth", v.kernel, &mod, &fn)) {
            emit_skip(test, v.label, "cubin or kernel missing");
            continue;
        }
        void *args[1] = {&out};
        const double us = time_kernel(g, fn, grid, 256, args);
        const double bytes = 64.0 * 2 * v.width * sizeof(float) * (double)threads;
        emit(test, v.label, "gbps", bytes / us / 1e3, us, grid);
        cuModuleUnload(mod);
    }
    cuMemFree(out);
}

void run_image_bandwidth(const Gpu &g)
{
    const char *test = "image_memory_bandwidth";
    constexpr int kW = 4096, kH = 4096, kFetch = 16;
    const unsigned grid = (unsigned)((uint64_t)kW * kH / kFetch / 256);
    const uint64_t threads = (uint64_t)grid * 256;
    CUDA_ARRAY_DESCRIPTOR ad = {};
    ad.Width = kW;
    ad.Height = kH;
    ad.Format = CU_AD_FORMAT_FLOAT;
    ad.NumChannels = 4;
    CUarray arr;
    DRV(cuArrayCreate(&arr, &ad));
    {
        std::vector<float> host((size_t)kW * kH * 4);
        fill_host(host.data(), host.size());
        CUDA_MEMCPY2D cp = {};
        cp.srcMemoryType = CU_MEMORYTYPE_HOST;
        cp.srcHost = host.data();
        cp.srcPitch = (size_t)kW * 16;
        cp.dstMemoryType = CU_MEMORYTYPE_ARRAY;
        cp.dstArray = arr;
        cp.WidthInBytes = (size_t)kW * 16;
        cp.Height = kH;
        DRV(cuMemcpy2D(&cp));
    }
    CUDA_RESOURCE_DESC rd = {};
    rd.resType = CU_RESOURCE_TYPE_ARRAY;
    rd.res.array.hArray = arr;
    CUDA_TEXTURE_DESC td = {};
    td.addressMode[0] = td.addressMode[1] = CU_TR_ADDRESS_MODE_CLAMP;
    td.filterMode = CU_TR_FILTER_MODE_POINT;
    CUtexObject tex = 0;
    DRV(cuTexObjectCreate(&tex, &rd, &td, nullptr));
    CUdeviceptr out = 0;
    DRV(cuMemAlloc(&out, threads * sizeof(float)));
    CUmodule mod;
    CUfunction fn;
    if (load_kernel(g, "image_bandwidth", "image_bandwidth", &mod, &fn)) {
        int w = kW, h = kH;
        void *args[4] = {&tex, &out, &w, &h};
        const double us = time_kernel(g, fn, grid, 256, args);
        emit(test, "float4", "gbps", (double)kFetch * 16.0 * (double)threads / us / 1e3, us, grid);
        cuModuleUnload(mod);
    } else {
        emit_skip(test, "float4", "cubin or kernel missing");
    }
    cuMemFree(out);
    cuTexObjectDestroy(tex);
    cuArrayDestroy(arr);
}

void run_kernel_latency(const Gpu &g)
{
    const char *test = "kernel_launch_latency";
    CUmodule mod;
    CUfunction fn;
    if (!load_kernel(g, "kernel_latency", "kernel_latency_noop", &mod, &fn)) {
        emit_skip(test, "roundtrip", "cubin or kernel missing");
        return;
    }
    void *args[1] = {nullptr};
    auto once = [&] {
        DRV(cuLaunchKernel(fn, 1, 1, 1, 1, 1, 1, 0, g.stream, args, nullptr));
        DRV(cuStreamSynchronize(g.stream));
    };
    for (unsigned w = 0; w < kWarmups; w++)
        once();
    constexpr unsigned kIters = 2000;
    double total_us = 0;
    for (unsigned i = 0; i < kIters; i++) {
        const auto t0 = std::chrono::steady_clock::now();
        once();
        const auto t1 = std::chrono::steady_clock::now();
        total_us += std::chrono::duration<double, std::micro>(t1 - t0).count();
    }
    emit(test, "roundtrip", "us", total_us / kIters, total_us / kIters, 1);
    cuModuleUnload(mod);
}

// ---- --dump: one launch of one reference kernel, output buffer written to a file ------------------

bool read_file(const char *path, std::vector<char> &bytes)
{
    std::FILE *f = std::fopen(path, "rb");
    if (!f)
        return false;
    std::fseek(f, 0, SEEK_END);
    const long n = std::ftell(f);
    std::fseek(f, 0, SEEK_SET);
    bytes.resize(n > 0 ? (size_t)n : 0);
    const bool ok = bytes.empty() || std::fread(bytes.data(), 1, bytes.size(), f) == bytes.size();
    std::fclose(f);
    return ok;
}

bool write_file(const char *path, const void *p, size_t n)
{
    std::FILE *f = std::fopen(path, "wb");
    if (!f)
        return false;
    const bool ok = std::fwrite(p, 1, n, f) == n;
    return std::fclose(f) == 0 && ok;
}

struct DumpArgs {
    const char *row = nullptr, *out = nullptr, *input = nullptr;
    unsigned blocks = 2;
    bool have_arg = false;
    double arg = 0;
    int w = 0, h = 0;
};

int launch_and_dump(const Gpu &g, CUfunction fn, unsigned grid, unsigned block, void **args, CUdeviceptr out,
                    size_t out_bytes, const char *path)
{
    DRV(cuMemsetD8(out, 0xA5, out_bytes));       // a kernel that writes nothing cannot pass for one that does
    DRV(cuLaunchKernel(fn, grid, 1, 1, block, 1, 1, 0, g.stream, args, nullptr));
    DRV(cuStreamSynchronize(g.stream));
    std::vector<char> host(out_bytes);
    DRV(cuMemcpyDtoH(host.data(), out, out_bytes));
    if (!write_file(path, host.data(), out_bytes)) {
        std::fprintf(stderr, "cannot write %s\n", path);
        return 5;
    }
    std::printf("{\"dump\": \"%s\", \"grid\": %u, \"block\": %u, \"bytes\": %zu}\n", path, grid, block, out_bytes);
    return 0;
}

int run_dump(const Gpu &g, const DumpArgs &d)
{
    const std::string row = d.row;
    const size_t slash = row.find('/');
    if (slash == std::string::npos) {
        std::fprintf(stderr, "--dump wants <test>/<label>\n");
        return 2;
    }
    const std::string test = row.substr(0, slash), label = row.substr(slash + 1);
    CUmodule mod;
    CUfunction fn;
    std::vector<char> input;
    if (d.input && !read_file(d.input, input)) {
        std::fprintf(stderr, "cannot read %s\n", d.input);
        return 5;
    }
    const int width = label == "float" ? 1 : label == "float2" ? 2 : label == "float4" ? 4 : 0;
    int rc = 2;

    if (test == "global_memory_bandwidth" && width) {
        const size_t in_bytes = (size_t)d.blocks * 256 * 16 * width * sizeof(float);
        if (input.size() != in_bytes) {
            std::fprintf(stderr, "--input must hold %zu bytes for %u blocks\n", in_bytes, d.blocks);
            return 2;
        }
        const std::string kernel = "global_bandwidth_v" + std::to_string(width);
        if (!load_kernel(g, "global_bandwidth", kernel.c_str(), &mod, &fn))
            return 6;
        CUdeviceptr in = 0, out = 0;
        const size_t out_bytes = (size_t)d.blocks * 256 * sizeof(float);
        DRV(cuMemAlloc(&in, in_bytes));
        DRV(cuMemAlloc(&out, out_bytes));
        DRV(cuMemcpyHtoD(in, input.data(), in_bytes));
        void *args[2] = {&in, &out};
        rc = launch_and_dump(g, fn, d.blocks, 256, args, out, out_bytes, d.out);
        cuMemFree(in);
        cuMemFree(out);
    } else if (test == "local_memory_bandwidth" && width) {
        const std::string kernel = "local_bandwidth_v" + std::to_string(width);
        if (!load_kernel(g, "local_bandwidth", kernel.c_str(), &mod, &fn))
            return 6;
        CUdeviceptr out = 0;
        const size_t out_bytes = (size_t)d.blocks * 256 * sizeof(float);
        DRV(cuMemAlloc(&out, out_bytes));
        void *args[1] = {&out};
        rc = launch_and_dump(g, fn, d.blocks, 256, args, out, out_bytes, d.out);
        cuMemFree(out);
    } else if (test == "image_memory_bandwidth" && width == 4) {
        const size_t texels = (size_t)d.w * d.h;
        if (d.w <= 0 || d.h <= 0 || texels % (16 * 256) != 0 || input.size() != texels * 16) {
            std::fprintf(stderr, "--dim W H with W*H a multiple of 4096, --input of W*H*16 bytes\n");
            return 2;
        }
        if (!load_kernel(g, "image_bandwidth", "image_bandwidth", &mod, &fn))
            return 6;
        CUDA_ARRAY_DESCRIPTOR ad = {};
        ad.Width = (size_t)d.w;
        ad.Height = (size_t)d.h;
        ad.Format = CU_AD_FORMAT_FLOAT;
        ad.NumChannels = 4;
        CUarray arr;
        DRV(cuArrayCreate(&arr, &ad));
        CUDA_MEMCPY2D cp = {};
        cp.srcMemoryType = CU_MEMORYTYPE_HOST;
        cp.srcHost = input.data();
        cp.srcPitch = (size_t)d.w * 16;
        cp.dstMemoryType = CU_MEMORYTYPE_ARRAY;
        cp.dstArray = arr;
        cp.WidthInBytes = (size_t)d.w * 16;
        cp.Height = (size_t)d.h;
        DRV(cuMemcpy2D(&cp));
        CUDA_RESOURCE_DESC rd = {};
        rd.resType = CU_RESOURCE_TYPE_ARRAY;
        rd.res.array.hArray = arr;
        CUDA_TEXTURE_DESC td = {};
        td.addressMode[0] = td.addressMode[1] = CU_TR_ADDRESS_MODE_CLAMP;
        td.filterMode = CU_TR_FILTER_MODE_POINT;
        CUtexObject tex = 0;
        DRV(cuTexObjectCreate(&tex, &rd, &td, nullptr));
        const unsigned grid = (unsigned)(texels / 16 / 256);
        const size_t out_bytes = (size_t)grid * 256 * sizeof(float);
        CUdeviceptr out = 0;
        DRV(cuMemAlloc(&out, out_bytes));
        int w = d.w, h = d.h;
        void *args[4] = {&tex, &out, &w, &h};
        rc = launch_and_dump(g, fn, grid, 256, args, out, out_bytes, d.out);
        cuMemFree(out);
        cuTexObjectDestroy(tex);
        cuArrayDestroy(arr);
    } else {
        const ComputeRow *r = nullptr;
        for (const ComputeRow &c : kComputeRows)
            if (test == c.test && label == c.label && !c.skip && c.block == 256)
                r = &c;
        if (!r) {
            std::fprintf(stderr, "no dumpable row %s\n", d.row);
            return 2;
        }
        if (!load_kernel(g, r->module, r->kernel, &mod, &fn))
            return 6;
        const size_t out_bytes = (size_t)d.blocks * r->out_per_block * r->elem_bytes;
        CUdeviceptr out = 0;
        DRV(cuMemAlloc(&out, out_bytes));
        const double a = d.have_arg ? d.arg : r->arg;
        float af = (float)a;
        double ad = a;
        int ai = (int)(long long)a;
        void *scalar = r->arg_kind == Arg::F32 ? (void *)&af : r->arg_kind == Arg::F64 ? (void *)&ad : (void *)&ai;
        void *args[2] = {&out, scalar};
        rc = launch_and_dump(g, fn, d.blocks, r->block, args, out, out_bytes, d.out);
        cuMemFree(out);
    }
    cuModuleUnload(mod);
    return rc;
}

const char *category_of(const std::string &unit)
{
    if (unit == "gflops" || unit == "tflops")
        return "fp_compute";
    if (unit == "gops" || unit == "tops")
        return "int_compute";
    if (unit == "gbps")
        return "bandwidth";
    return "latency";
}

bool write_csv(const char *path, const char *device, int driver)
{
    std::FILE *f = std::fopen(path, "w");
    if (!f)
        return false;
    std::fprintf(f, "format_version,backend,platform,device,driver,category,test,metric,unit,status,value,reason,"
                    "display,description,metric_description\n");
    for (const CsvRow &r : g_rows) {
        std::fprintf(f, "2,CUDA,CUDA,\"%s\",%d.%d,%s,%s,%s,%s,", device, driver / 1000, driver % 1000 / 10,
                     category_of(r.unit), r.test.c_str(), r.label.c_str(), r.unit.c_str());
        if (r.ok)
            std::fprintf(f, "ok,%.4f,,,,\n", r.value);
        else
            std::fprintf(f, "unsupported,,\"%s\",,,\n", r.reason.c_str());
    }
    return std::fclose(f) == 0;
}

} // namespace

int main(int argc, char **argv)
{
    if (argc < 2) {
        std::fprintf(stderr, "usage: %s <cubin dir> [--budget-us N] [--filter substring] [--csv file]\n"
                             "       %s <cubin dir> --dump <test>/<label> <out file> [--blocks N] [--arg X] [--input file] [--dim W H]\n",
                     argv[0], argv[0]);
        return 2;
    }
    Gpu g;
    g.dir = argv[1];
    const char *filter = nullptr, *csv = nullptr;
    DumpArgs dump;
    for (int i = 2; i < argc; i++) {
        const bool has_value = i + 1 < argc;
        if (!std::strcmp(argv[i], "--dump") && i + 2 < argc) {
            dump.row = argv[++i];
            dump.out = argv[++i];
        } else if (!std::strcmp(argv[i], "--blocks") && has_value && std::atol(argv[i + 1]) > 0 &&
                   std::atol(argv[i + 1]) <= 65536)
            dump.blocks = (unsigned)std::atol(argv[++i]);
        else if (!std::strcmp(argv[i], "--arg") && has_value) {
            dump.have_arg = true;
            dump.arg = std::strtod(argv[++i], nullptr);
        } else if (!std::strcmp(argv[i], "--input") && has_value)
            dump.input = argv[++i];
        else if (!std::strcmp(argv[i], "--dim") && i + 2 < argc) {
            dump.w = std::atoi(argv[++i]);
            dump.h = std::atoi(argv[++i]);
        } else if (!std::strcmp(argv[i], "--budget-us") && has_value && std::atol(argv[i + 1]) > 0)
            g.budget_us = (unsigned)std::atol(argv[++i]);
        else if (!std::strcmp(argv[i], "--filter") && has_value)
            filter = argv[++i];
        else if (!std::strcmp(argv[i], "--csv") && has_value)
            csv = argv[++i];
        else {
            std::fprintf(stderr, "unknown or incomplete argument: %s\n", argv[i]);
            return 2;
        }
    }
    if (filter && !filter[0])
        filter = nullptr;

    DRV(cuInit(0));
    DRV(cuDeviceGet(&g.dev, 0));
    DRV(cuDevicePrimaryCtxRetain(&g.ctx, g.dev));
    DRV(cuCtxSetCurrent(g.ctx));
    DRV(cuStreamCreate(&g.stream, CU_STREAM_NON_BLOCKING));
    DRV(cuDeviceGetAttribute(&g.sms, CU_DEVICE_ATTRIBUTE_MULTIPROCESSOR_COUNT, g.dev));
    DRV(cuDeviceTotalMem(&g.vram, g.dev));
    int major = 0, minor = 0;
    DRV(cuDeviceGetAttribute(&major, CU_DEVICE_ATTRIBUTE_COMPUTE_CAPABILITY_MAJOR, g.dev));
    DRV(cuDeviceGetAttribute(&minor, CU_DEVICE_ATTRIBUTE_COMPUTE_CAPABILITY_MINOR, g.dev));
    if (major != 10) {
        std::fprintf(stderr, "the cubins are built for sm_100a; this device is sm_%d%d\n", major, minor);
        return 4;
    }

    if (dump.row) {
        const int drc = run_dump(g, dump);
        cuStreamDestroy(g.stream);
        cuDevicePrimaryCtxRelease(g.dev);
        return drc;
    }

    if (wanted(filter, "global_memory_bandwidth", "float float2 float4"))
        run_global_bandwidth(g, filter && std::strstr("global_memory_bandwidth", filter) ? nullptr : filter);
    if (wanted(filter, "local_memory_bandwidth", "float float2 float4"))
        run_local_bandwidth(g, filter && std::strstr("local_memory_bandwidth", filter) ? nullptr : filter);
    if (wanted(filter, "image_memory_bandwidth", "float4"))
        run_image_bandwidth(g);
    for (const ComputeRow &r : kComputeRows)
        if (wanted(filter, r.test, r.label))
            run_compute(g, r);
    if (wanted(filter, "kernel_launch_latency", "roundtrip"))
        run_kernel_latency(g);

    int rc = 0;
    if (csv) {
        char name[256] = "";
        int driver = 0;
        DRV(cuDeviceGetName(name, sizeof name, g.dev));
        DRV(cuDriverGetVersion(&driver));
        if (!write_csv(csv, name, driver)) {
            std::fprintf(stderr, "cannot write %s\n", csv);
            rc = 5;
        }
    }
    cuStreamDestroy(g.stream);
    cuDevicePrimaryCtxRelease(g.dev);
    return rc;
}
