// CudaPeak for B200: device enumeration, the concurrent multi-GPU driver and the
// tests of the CUDA slot, all on top of the kernel shim.
//
// Run model.  The reference visits devices one after another in the calling
// thread (src/cuda/cuda_peak.cpp:129-205).  Here every selected GPU gets its own
// host thread, context and stream; the threads walk the same test list and meet
// at a start gate before each test, so the GPUs of a box are loaded at the same
// time.  Workers only *produce* readings; the calling thread alone talks to the
// logger (one open test at a time, FFI callbacks on the launching thread): it
// opens device scopes in index order, streams the first device's readings as they
// arrive and replays the others, then adds a box-aggregate pseudo device when
// more than one GPU ran.  Nothing is exchanged between GPUs: replicas only.
#include <algorithm>
#include <atomic>
#include <chrono>
#include <cmath>
#include <condition_variable>
#include <cstring>
#include <deque>
#include <functional>
#include <mutex>
#include <sstream>
#include <thread>

#include <cuda/cuda_peak.h>
#include <common/common.h>
#include <common/options.h>

#include "host_check.hpp"
#include "start_gate.hpp"

namespace {

// Datasheet peaks used for the "% of spec" notes: NVIDIA HGX B200 (8-GPU board)
// figures divided by eight, dense (the sheet's headline numbers include 2:4 sparsity).
constexpr double kSpecHbmGBps = 8000.0;
constexpr double kSpecBf16Tflops = 2250.0;
constexpr double kSpecFp8Tflops = 4500.0;
constexpr double kSpecFp4Tflops = 9000.0;
constexpr double kSpecInt8Tops = 4500.0;
constexpr double kSpecFp32Gflops = 80000.0;
constexpr double kSpecFp64Tflops = 37.0;    // HGX B200: 296 TFLOPS FP64 tensor core per board

std::string pct(double value, double peak, const char *what)
{
    std::ostringstream ss;
    ss.setf(std::ios::fixed);
    ss.precision(1);
    ss << 100.0 * value / peak << "% of the " << what << " datasheet peak (" << (long long)peak << ").";
    return ss.str();
}

// "... N cycles per instruction at X MHz": the kernel's own clock64 / %globaltimer span of CTA 0 turns the
// measured time into tensor-core cycles, which separates the instruction rate from the clock the power cap allows.
std::string cyclesNote(double secondsPerLaunch, const unsigned long long clock[2], double instructionsPerSm)
{
    if (clock[1] == 0 || instructionsPerSm <= 0)
        return "";
    const double mhz = (double)clock[0] / (double)clock[1] * 1e3;
    std::ostringstream ss;
    ss.setf(std::ios::fixed);
    ss.precision(1);
    ss << "  About " << secondsPerLaunch * mhz * 1e6 / instructionsPerSm << " cycles per instruction (128 is the tensor core's rate) at the "
       << (long long)(mhz + 0.5) << " MHz the SMs ran at under the power cap.";
    return ss.str();
}

std::string shimError(const char *what)
{
    return std::string(what) + ": " + clpk_last_error();
}

struct DeviceBuffer {
    void *p = nullptr;
    ~DeviceBuffer() { clpk_free(p); }
    bool alloc(size_t bytes) { return clpk_malloc(&p, bytes) == CLPK_OK; }
    template <typename T> T *as() const { return static_cast<T *>(p); }
};

struct PinnedBuffer {
    void *p = nullptr;
    ~PinnedBuffer() { clpk_free_host(p); }
    bool alloc(size_t bytes) { return clpk_malloc_host(&p, bytes) == CLPK_OK; }
};

} // namespace

// ---------------------------------------------------------------------------------
// Worker: one GPU, one host thread
// ---------------------------------------------------------------------------------

struct B200Worker {
    int device = 0;
    cuda_device_info_t info;
    void *stream = nullptr;
    unsigned warmup = 2, targetUs = DEFAULT_TARGET_TIME_US, forcedIters = 0;
    unsigned latencyIters = 2000;
    // The device threads meet here immediately before every timed batch (after this GPU's warm-ups
    // and probe launch), so that the timed regions of all GPUs overlap and every GPU is measured
    // under the power and thermal load of a full box.  Null when a single GPU runs.
    StartGate *batchGate = nullptr;
    std::chrono::milliseconds batchGateTimeout{20000};

    // results handed to the calling thread, in plan order
    std::mutex m;
    std::condition_variable cv;
    std::deque<B200TestResult> ready;
    bool finished = false;
    std::string fatal;

    // Mirrors CudaPeak::runKernel (src/cuda/cuda_peak.cpp:64-107): untimed
    // warm-ups, one timed probe launch, iters from pickIters, one timed batch.
    // Returns seconds per launch, negative on error (message in err).
    double timeLaunches(const std::function<int()> &launch, std::string &err) const
    {
        void *e0 = nullptr, *e1 = nullptr;
        if (clpk_event_create(&e0) != CLPK_OK || clpk_event_create(&e1) != CLPK_OK) {
            err = shimError("event create");
            return -1.0;
        }
        auto batch = [&](unsigned n, float &ms) -> bool {
            if (clpk_event_record(e0, stream) != CLPK_OK) return false;
            for (unsigned i = 0; i < n; ++i)
                if (launch() != CLPK_OK) return false;
            if (clpk_event_record(e1, stream) != CLPK_OK || clpk_event_sync(e1) != CLPK_OK) return false;
            return clpk_event_elapsed_ms(e0, e1, &ms) == CLPK_OK;
        };
        double result = -1.0;
        do {
            bool ok = true;
            for (unsigned w = 0; w < warmup && ok; ++w)
                ok = launch() == CLPK_OK && clpk_stream_sync(stream) == CLPK_OK;
            float ms = 0;
            if (!ok || !batch(1, ms)) break;
            const unsigned iters = pickIters((double)ms * 1000.0, targetUs, forcedIters);
            if (batchGate)
                batchGate->arrive(batchGateTimeout);
            if (!batch(iters, ms)) break;
            result = (double)ms * 1e-3 / iters;
        } while (false);
        if (result < 0)
            err = shimError("launch");
        clpk_event_destroy(e0);
        clpk_event_destroy(e1);
        return result;
    }

    void push(B200TestResult &&r)
    {
        {
            std::lock_guard<std::mutex> lk(m);
            ready.push_back(std::move(r));
        }
        cv.notify_all();
    }
};

// ---------------------------------------------------------------------------------
// The tests
// ---------------------------------------------------------------------------------

struct B200Harness {
    using Test = std::function<void(B200Worker &, B200TestResult &)>;

    static B200Reading ok(const std::string &metric, double value, const std::string &info, double work = 0,
                          double seconds = 0)
    {
        B200Reading r;
        r.metric = metric;
        r.value = (float)value;
        r.info = info;
        r.work = work;
        r.seconds = seconds;
        return r;
    }

    static B200Reading bad(const std::string &metric, ResultStatus st, const std::string &reason,
                           const std::string &info = "")
    {
        B200Reading r;
        r.metric = metric;
        r.status = st;
        r.reason = reason;
        r.info = info;
        return r;
    }

    // ---- fp32 chains ------------------------------------------------------------------

    static void computeSP(B200Worker &w, B200TestResult &out)
    {
        out.spec = {"single_precision_compute", "Single-precision compute", "gflops", Category::Unknown,
                    "Peak arithmetic speed of the GPU's shader cores on 32-bit fractional numbers -- the ordinary "
                    "float type.  Nothing touches memory, so only the arithmetic units limit the rate."};
        const char *refNote = "clpeak's chain x = x*x + c, 4096 operations per thread, outputs compared with the "
                              "same chain on the host.";
        const char *seedNote = "2^20 work-items, each a float4 drawn uniform[-1,1) from seed 0, 4096 steps of "
                               "x = x*y + x with y = 0.999; every output compared with the host.";
        // reference geometry: numSMs*2048*256 threads, capped by a quarter of VRAM (compute_kernel.cpp:49-57)
        uint64_t blocks = targetGlobalThreads((uint32_t)w.info.numSMs) / 256;
        blocks = std::min<uint64_t>(blocks, w.info.totalGlobalMem / 4 / (256 * sizeof(float)));
        DeviceBuffer buf;
        if (!buf.alloc(blocks * 256 * sizeof(float))) {
            out.readings.push_back(bad("float", ResultStatus::Error, "Failed to allocate output buffer", refNote));
        } else {
            std::string err;
            const float a = 1.3f;
            double s = w.timeLaunches([&] { return clpk_compute_sp(buf.as<float>(), a, (uint32_t)blocks, w.stream); }, err);
            if (s < 0) {
                out.readings.push_back(bad("float", ResultStatus::Error, err, refNote));
            } else {
                std::vector<float> head(512);
                clpk_memcpy_d2h(head.data(), buf.p, head.size() * sizeof(float), w.stream);
                clpk_stream_sync(w.stream);
                bool same = true;
                for (size_t i = 0; i < head.size() && same; ++i)
                    same = b200check::sameFloat(head[i], b200check::chainReference(a, (unsigned)(i % 256)));
                const double work = (double)blocks * 256.0 * COMPUTE_FP_WORK_PER_WI;
                const double gflops = work / s / 1e9;
                if (!same)
                    out.readings.push_back(bad("float", ResultStatus::Error, "output differs from the host chain", refNote));
                else
                    out.readings.push_back(ok("float", gflops, std::string(refNote) + "  " + pct(gflops, kSpecFp32Gflops, "fp32 GFLOPS"), work, s));
            }
        }
        // seeded chain of the CPU-runnable baseline pair
        const uint64_t items = 1ull << 20;
        DeviceBuffer sb;
        if (!sb.alloc(items * sizeof(float))) {
            out.readings.push_back(bad("float4_seeded", ResultStatus::Error, "Failed to allocate output buffer", seedNote));
            return;
        }
        std::string err;
        double s = w.timeLaunches([&] { return clpk_mad_chain(sb.as<float>(), items, 0, 0.999f, 4096, w.stream); }, err);
        if (s < 0) {
            out.readings.push_back(bad("float4_seeded", ResultStatus::Error, err, seedNote));
            return;
        }
        std::vector<float> got(4096);
        clpk_memcpy_d2h(got.data(), sb.p, got.size() * sizeof(float), w.stream);
        clpk_stream_sync(w.stream);
        bool same = true;
        for (size_t i = 0; i < got.size() && same; ++i)
            same = b200check::sameFloat(got[i], b200check::seededChain(0, i, 0.999f, 4096));
        // the finite-range prefix (64 steps) has real values, not just infinities
        if (same && clpk_mad_chain(sb.as<float>(), items, 0, 0.999f, 64, w.stream) == CLPK_OK) {
            clpk_memcpy_d2h(got.data(), sb.p, got.size() * sizeof(float), w.stream);
            clpk_stream_sync(w.stream);
            for (size_t i = 0; i < got.size() && same; ++i)
                same = std::isfinite(got[i]) && b200check::sameFloat(got[i], b200check::seededChain(0, i, 0.999f, 64));
        }
        const double work = (double)items * 4 * 4096 * 2;
        if (!same)
            out.readings.push_back(bad("float4_seeded", ResultStatus::Error, "output differs from the host chain", seedNote));
        else
            out.readings.push_back(ok("float4_seeded", work / s / 1e9, seedNote, work, s));
    }

    // ---- chains of the other element types -------------------------------------------------

    struct ChainVariant { int chain; const char *metric; const char *note; };
    struct ChainTest {
        const char *tag, *title, *unit, *desc;
        double start;                        // the scalar the reference's host code passes
        std::vector<ChainVariant> variants;
    };

    static const std::vector<ChainTest> &chainTests()
    {
        static const char *w1 = "One value per thread at a time -- the plain, unvectorised case.";
        static const char *w2 = "Two values per thread at a time, packed into one instruction.";
        static const std::vector<ChainTest> tests = {
            {"half_precision_compute", "Half-precision compute", "gflops",
             "Peak arithmetic speed on 16-bit fractional numbers -- half the size of a normal float, and what graphics "
             "and on-device AI mostly run on.  NVIDIA shader cores reach full speed only on the packed form that does "
             "two at a time.",
             1.3, {{CLPK_CHAIN_HALF, "half", w1}, {CLPK_CHAIN_HALF2, "half2", w2}}},
            {"double_precision_compute", "Double-precision compute", "gflops",
             "Peak arithmetic speed on 64-bit fractional numbers, the high-accuracy type scientific computing relies "
             "on.  Consumer GeForce cards run these dozens of times slower than 32-bit; the datacenter parts do not.",
             1.3, {{CLPK_CHAIN_DOUBLE, "double", ""}}},
            {"mixed_precision_compute", "Mixed-precision compute fp16xfp16+fp32", "gflops",
             "Peak speed when the GPU multiplies 16-bit numbers but keeps the running total in 32 bits -- the "
             "accuracy-preserving pattern AI code uses.  This is the shader cores, not the tensor cores.",
             1.3, {{CLPK_CHAIN_MIXED, "mp", ""}}},
            {"bfloat16_compute", "BF16 compute bf16xbf16+fp32", "gflops",
             "Peak speed on bfloat16 -- 16 bits arranged for AI work, trading digits of accuracy for the number range "
             "of a full float.  Again the shader cores, with the tensor-core figure in the tcgen05 rows.",
             1.3, {{CLPK_CHAIN_BF16, "bf16", ""}}},
            {"integer_compute", "Integer compute (32-bit IMAD)", "gops",
             "Peak speed on 32-bit whole numbers -- the arithmetic behind indexing, addressing and bit manipulation, "
             "which shaders do alongside their fractional maths.",
             3, {{CLPK_CHAIN_INT32, "int", ""}}},
            {"integer_compute_int8_dp", "INT8 dot-product compute (__dp4a)", "gops",
             "Peak speed of the 8-bit dot-product instruction, which multiplies four pairs of small whole numbers and "
             "sums them in one step -- the shader-core path for quantized (compressed) neural networks.",
             4, {{CLPK_CHAIN_INT8_DOT1, "int8_dp", "One chain of dot products, each waiting on the one before it."},
                 {CLPK_CHAIN_INT8_DOT2, "int8_dp2", "Two independent chains, so the GPU has a second dot product to get on with while the first is still finishing."},
                 {CLPK_CHAIN_INT8_DOT4, "int8_dp4", "Four independent chains."},
                 {CLPK_CHAIN_INT8_DOT8, "int8_dp8", "Eight independent chains.  Where this stops improving on four, the hardware itself is the limit, not the waiting."}}},
        };
        return tests;
    }

    static void typedChain(B200Worker &w, B200TestResult &out, const ChainTest &t)
    {
        out.spec = {t.tag, t.title, t.unit, Category::Unknown, t.desc};
        for (const ChainVariant &v : t.variants) {
            const std::string note = std::string(v.note) + (v.note[0] ? "  " : "") +
                                     "Outputs of the first two blocks compared with the same chain on the host.";
            uint32_t ops = 0, elem = 4;
            clpk_compute_chain_info(v.chain, &ops, &elem);
            // reference geometry: numSMs*2048*256 threads, capped by a quarter of VRAM (compute_kernel.cpp:49-57)
            uint64_t blocks = targetGlobalThreads((uint32_t)w.info.numSMs) / 256;
            blocks = std::min<uint64_t>(blocks, w.info.totalGlobalMem / 4 / (256ull * elem));
            DeviceBuffer buf;
            if (!buf.alloc(blocks * 256 * elem)) {
                out.readings.push_back(bad(v.metric, ResultStatus::Error, "Failed to allocate output buffer", note));
                continue;
            }
            std::string err;
            const double s = w.timeLaunches([&] { return clpk_compute_chain(v.chain, buf.p, t.start, (uint32_t)blocks, w.stream); }, err);
            if (s < 0) {
                out.readings.push_back(bad(v.metric, ResultStatus::Error, err, note));
                continue;
            }
            std::vector<uint8_t> head(512 * (size_t)elem);
            clpk_memcpy_d2h(head.data(), buf.p, head.size(), w.stream);
            clpk_stream_sync(w.stream);
            bool same = true;
            for (unsigned i = 0; i < 512 && same; ++i) {
                uint64_t got = 0;
                std::memcpy(&got, head.data() + (size_t)i * elem, elem);
                same = got == b200check::typedChainBits(v.chain, t.start, i % 256);
            }
            const double work = (double)blocks * 256.0 * ops;
            if (!same)
                out.readings.push_back(bad(v.metric, ResultStatus::Error, "output differs from the host chain", note));
            else
                out.readings.push_back(ok(v.metric, work / s / 1e9, note, work, s));
        }
    }

    // ---- tensor-core peak ----------------------------------------------------------------

    struct KindRow { int kind; const char *tag, *display, *metric, *unit; double spec; const char *specName; const char *desc; };

    static const std::vector<KindRow> &kindRows()
    {
        static const std::vector<KindRow> rows = {
            {CLPK_MMA_F16, "wmma_fp16", "tcgen05 fp16xfp16+fp32 128x256x16", "wmma_fp16", "tflops", kSpecBf16Tflops, "dense fp16 TFLOPS",
             "Peak speed of the tensor cores on 16-bit inputs with a 32-bit running total, issued as Blackwell tcgen05.mma "
             "instructions that accumulate in tensor memory.  This is the everyday precision of AI work."},
            {CLPK_MMA_F16_F16, "wmma_fp16_f16", "tcgen05 fp16xfp16+fp16 128x256x16", "fp16_f16acc", "tflops", kSpecBf16Tflops, "dense fp16 TFLOPS",
             "The same 16-bit tensor-core path keeping its running total in 16 bits as well -- cheaper to store, easier to overflow."},
            {CLPK_MMA_BF16, "wmma_bf16", "tcgen05 bf16xbf16+fp32 128x256x16", "wmma_bf16", "tflops", kSpecBf16Tflops, "dense bf16 TFLOPS",
             "Tensor cores on bfloat16 -- 16 bits arranged for AI work, trading digits of accuracy for the number range of a full float."},
            {CLPK_MMA_TF32, "wmma_tf32", "tcgen05 tf32xtf32+fp32 128x256x8", "wmma_tf32", "tflops", kSpecBf16Tflops / 2, "dense tf32 TFLOPS",
             "Tensor cores on TF32: 32-bit storage of which the multiplier reads 19 bits, NVIDIA's drop-in speed-up for float code."},
            {CLPK_MMA_E4M3, "wmma_fp8_e4m3", "tcgen05 FP8(E4M3)+fp32 128x256x32", "fp8_e4m3", "tflops", kSpecFp8Tflops, "dense fp8 TFLOPS",
             "Tensor cores on 8-bit numbers, in the variant that spends its bits on accuracy rather than range."},
            {CLPK_MMA_E5M2, "wmma_fp8_e5m2", "tcgen05 FP8(E5M2)+fp32 128x256x32", "fp8_e5m2", "tflops", kSpecFp8Tflops, "dense fp8 TFLOPS",
             "The same 8-bit tensor-core path in the variant that spends its bits on range rather than accuracy."},
            {CLPK_MMA_E2M1, "wmma_fp4_e2m1", "tcgen05 FP4(E2M1) unscaled 128x256x32", "fp4_e2m1", "tflops", kSpecFp8Tflops, "dense fp8 TFLOPS (this path runs at the 8-bit rate)",
             "4-bit numbers fed through the 8-bit tensor-core path without block scale factors: storage halves, speed does not."},
            {CLPK_MMA_MXF4, "wmma_mxf4_e2m1", "tcgen05 MXFP4(E2M1) block-scaled 128x256x64", "mxf4_e2m1", "tflops", kSpecFp4Tflops, "dense fp4 TFLOPS",
             "4-bit numbers with a shared scale factor per block of 32, the open MX format."},
            {CLPK_MMA_NVF4, "wmma_nvf4_e2m1", "tcgen05 NVFP4(E2M1) block-scaled 128x256x64", "nvf4_e2m1", "tflops", kSpecFp4Tflops, "dense fp4 TFLOPS",
             "NVIDIA's own 4-bit block format, with a finer scale factor shared by every 16 values instead of every 32."},
            {CLPK_MMA_I8, "wmma_int8_k32", "tcgen05 int8xint8+int32 128x256x32", "int8_k32", "tops", kSpecInt8Tops, "dense int8 TOPS",
             "Tensor cores on 8-bit whole numbers with 32-bit totals -- the format quantized neural networks use."},
        };
        return rows;
    }

    static void tensorPeak(B200Worker &w, B200TestResult &out, const KindRow &row)
    {
        out.spec = {row.tag, row.display, row.unit, Category::Unknown, row.desc};
        const int kind = row.kind;
        const int K = clpk_mma_kind_k(kind);
        const bool scaled = (kind == CLPK_MMA_MXF4 || kind == CLPK_MMA_NVF4);
        const uint32_t grid = 4u * (uint32_t)w.info.numSMs, nMma = 1u << 14;
        const std::string note = "2^14 instructions per CTA on " + std::to_string(grid) +
                                 " CTAs, operands seeded (uniform[-1,1) / N(0,1) quantised per block), final accumulator tile "
                                 "checked against the host.";
        auto fail = [&](const std::string &why) { out.readings.push_back(bad(row.metric, ResultStatus::Error, why, note)); };

        // operands: generated and quantised on the device, copied back for the check
        const size_t aBytes = 128 * 32, bBytes = 256 * 32;
        DeviceBuffer f32, dA, dB, dSfa, dSfb, dOut, dChk, dStatus, dClock;
        if (!f32.alloc(256 * 64 * sizeof(float)) || !dA.alloc(aBytes) || !dB.alloc(bBytes) || !dSfa.alloc(128 * 4) ||
            !dSfb.alloc(256 * 4) || !dOut.alloc(128 * 256 * 4) || !dChk.alloc(grid * 4) || !dStatus.alloc(4) || !dClock.alloc(16))
            return fail("Failed to allocate buffers");
        int rc = CLPK_OK;
        auto gen = [&](void *dst, void *sf, int rows, uint64_t first) {
            if (kind == CLPK_MMA_I8) {
                rc |= clpk_fill_i8(static_cast<int8_t *>(dst), (uint64_t)rows * K, 2 + first, w.stream);
                return;
            }
            if (!scaled) {
                rc |= clpk_fill_f32(f32.as<float>(), (uint64_t)rows * K, 2 + first, CLPK_DIST_UNIFORM_PM1, 0, 1, w.stream);
                const int dt = (kind == CLPK_MMA_F16 || kind == CLPK_MMA_F16_F16) ? CLPK_DT_F16 : kind == CLPK_MMA_BF16 ? CLPK_DT_BF16
                             : kind == CLPK_MMA_E4M3 ? CLPK_DT_E4M3 : kind == CLPK_MMA_TF32 ? CLPK_DT_TF32
                             : kind == CLPK_MMA_E2M1 ? CLPK_DT_E2M1 : CLPK_DT_E5M2;
                if (kind == CLPK_MMA_E2M1)      // spread over e2m1's +-6 range
                    rc |= clpk_fill_f32(f32.as<float>(), (uint64_t)rows * K, 2 + first, CLPK_DIST_NORMAL, 0, 2, w.stream);
                rc |= clpk_convert_f32(dst, f32.as<float>(), (uint64_t)rows * K, dt, w.stream);
                return;
            }
            rc |= clpk_fill_f32(f32.as<float>(), (uint64_t)rows * K, 3 + first, CLPK_DIST_NORMAL, 0, 1, w.stream);
            // N(0,1) tiles: |x| stays below ~5, so absmax/(6*448) is about 2^-9; a fixed power of two keeps the
            // tensor scale exact on both sides.
            rc |= clpk_quantize_fp4(static_cast<uint8_t *>(dst), static_cast<uint8_t *>(sf), f32.as<float>(), rows, K,
                                    kind == CLPK_MMA_MXF4 ? CLPK_DT_MXF4 : CLPK_DT_NVF4,
                                    kind == CLPK_MMA_MXF4 ? 1.0f : 0.001953125f, w.stream);
        };
        gen(dA.p, dSfa.p, 128, 0);
        gen(dB.p, dSfb.p, 256, 1);
        if (rc != CLPK_OK)
            return fail(shimError("operand generation"));

        clpk_mma_peak_args_t a{};
        a.kind = kind;
        a.d_a = dA.p; a.d_b = dB.p; a.d_sfa = dSfa.p; a.d_sfb = dSfb.p;
        a.n_mma = nMma; a.grid = grid; a.n_out_tiles = 1;
        a.d_out = dOut.p; a.d_checksum = dChk.as<uint32_t>(); a.d_status = dStatus.as<uint32_t>();
        a.d_clock = dClock.as<unsigned long long>();
        clpk_memset(dClock.p, 0, 16, w.stream);

        std::string err;
        const double s = w.timeLaunches([&] { return clpk_mma_peak(&a, w.stream); }, err);
        if (s < 0)
            return fail(err);

        std::vector<uint8_t> hA(aBytes), hB(bBytes), hSfa(128 * 4), hSfb(256 * 4);
        std::vector<uint32_t> tile(128 * 256), chk(grid);
        uint32_t status = 0;
        unsigned long long clock[2] = {0, 0};
        clpk_memcpy_d2h(clock, dClock.p, sizeof clock, w.stream);
        clpk_memcpy_d2h(hA.data(), dA.p, aBytes, w.stream);
        clpk_memcpy_d2h(hB.data(), dB.p, bBytes, w.stream);
        clpk_memcpy_d2h(hSfa.data(), dSfa.p, hSfa.size(), w.stream);
        clpk_memcpy_d2h(hSfb.data(), dSfb.p, hSfb.size(), w.stream);
        clpk_memcpy_d2h(tile.data(), dOut.p, tile.size() * 4, w.stream);
        clpk_memcpy_d2h(chk.data(), dChk.p, chk.size() * 4, w.stream);
        clpk_memcpy_d2h(&status, dStatus.p, 4, w.stream);
        if (clpk_stream_sync(w.stream) != CLPK_OK)
            return fail(shimError("read back"));
        if (status != 0)
            return fail("a device-side wait timed out (status " + std::to_string(status) + ")");
        for (uint32_t c : chk)
            if (c != chk[0])
                return fail("CTAs disagree on the accumulator checksum");
        double worst = 0;
        std::string verdict;
        if (kind == CLPK_MMA_F16_F16) {
            // 2^14 additions saturate a 16-bit running total; the arithmetic is checked on one instruction
            a.n_mma = 1;
            a.grid = 1;
            if (clpk_mma_peak(&a, w.stream) != CLPK_OK)
                return fail(shimError("single-instruction launch"));
            clpk_memcpy_d2h(tile.data(), dOut.p, tile.size() * 4, w.stream);
            if (clpk_stream_sync(w.stream) != CLPK_OK)
                return fail(shimError("read back"));
            verdict = b200check::checkHalfAccumTile(hA.data(), hB.data(), tile.data(), &worst);
        } else {
            verdict = b200check::checkTile(kind, hA.data(), hB.data(), hSfa.data(), hSfb.data(), nMma, tile.data(), &worst);
        }
        if (!verdict.empty())
            return fail("accumulator check failed: " + verdict);

        const double work = clpk_mma_flops_per_instr(kind) * nMma * grid;
        const double t = work / s / 1e12;
        out.readings.push_back(ok(row.metric, t, note + "  " + pct(t, row.spec, row.specName) +
                                                     cyclesNote(s, clock, (double)nMma * grid / w.info.numSMs), work, s));
    }

    // 2:4 structured-sparse kinds (tcgen05.mma.sp): a dense float tile is generated on the device, pruned on the
    // host (the selection is data dependent and tiny), and the compressed tile goes back for quantisation.
    static const std::vector<KindRow> &sparseRows(bool integer)
    {
        static const std::vector<KindRow> fp = {
            {CLPK_MMA_E4M3_SP, "wmma_fp8_e4m3_sparse", "tcgen05 FP8(E4M3) 2:4 sparse 128x256x64", "fp8_e4m3_sparse", "tflops", 2 * kSpecFp8Tflops, "sparse fp8 TFLOPS",
             "8-bit tensor cores with structured sparsity: of every four values along a row of one input two are zero and "
             "are skipped, which doubles the nominal rate.  Work is counted as if the zeros were multiplied."},
            {CLPK_MMA_MXF4_SP, "wmma_mxf4_sparse", "tcgen05 MXFP4 2:4 sparse 128x256x128", "mxf4_sparse", "tflops", 2 * kSpecFp4Tflops, "sparse fp4 TFLOPS",
             "The 4-bit MX format combined with structured sparsity (two of every four pairs kept)."},
            {CLPK_MMA_NVF4_SP, "wmma_nvf4_sparse", "tcgen05 NVFP4 2:4 sparse 128x256x128", "nvf4_sparse", "tflops", 2 * kSpecFp4Tflops, "sparse fp4 TFLOPS",
             "NVIDIA's 4-bit block format combined with structured sparsity -- the highest nominal rate of the chip."},
        };
        static const std::vector<KindRow> in = {
            {CLPK_MMA_I8_SP, "wmma_int8_sparse", "tcgen05 int8 2:4 sparse 128x256x64", "int8_sparse", "tops", 2 * kSpecInt8Tops, "sparse int8 TOPS",
             "8-bit whole-number tensor cores with structured sparsity: two of every four values of one input are zero and skipped."},
        };
        return integer ? in : fp;
    }

    static void tensorSparse(B200Worker &w, B200TestResult &out, const KindRow &row)
    {
        out.spec = {row.tag, row.display, row.unit, Category::Unknown, row.desc};
        const int kind = row.kind;
        const int K = b200check::sparseK(kind);
        const bool fp4 = K == 128;
        const int nsf = kind == CLPK_MMA_NVF4_SP ? 4 : 2;
        const uint32_t grid = 4u * (uint32_t)w.info.numSMs, nMma = 1u << 14;
        const std::string note = "2^14 instructions per CTA on " + std::to_string(grid) +
                                 " CTAs, work counted at the logical K=" + std::to_string(K) +
                                 "; seeded A pruned 2:4 by magnitude, final accumulator tile checked against the host.";
        auto fail = [&](const std::string &why) { out.readings.push_back(bad(row.metric, ResultStatus::Error, why, note)); };

        const size_t aBytes = 128 * 32, bBytes = 256 * 64, metaBytes = 128 * 8;   // K/2 x 8-bit = K/2 x 2 x 4-bit
        DeviceBuffer f32, dA, dB, dSfa, dSfb, dMeta, dOut, dChk, dStatus, dClock;
        if (!f32.alloc(256 * 128 * sizeof(float)) || !dA.alloc(aBytes) || !dB.alloc(bBytes) || !dSfa.alloc(128 * 4) ||
            !dSfb.alloc(256 * 4) || !dMeta.alloc(metaBytes) || !dOut.alloc(128 * 256 * 4) || !dChk.alloc(grid * 4) || !dStatus.alloc(4) ||
            !dClock.alloc(16))
            return fail("Failed to allocate buffers");

        // A: dense on the device -> host prune -> compressed floats back -> device quantise
        std::vector<float> dense(128 * (size_t)K), comp;
        std::vector<uint8_t> meta;
        int rc = CLPK_OK;
        if (kind == CLPK_MMA_I8_SP) {
            std::vector<int8_t> raw(dense.size());
            rc |= clpk_fill_i8(f32.as<int8_t>(), raw.size(), 2, w.stream);
            rc |= clpk_memcpy_d2h(raw.data(), f32.p, raw.size(), w.stream);
            rc |= clpk_stream_sync(w.stream);
            for (size_t i = 0; i < raw.size(); ++i)
                dense[i] = (float)raw[i];
        } else {
            rc |= clpk_fill_f32(f32.as<float>(), dense.size(), fp4 ? 3 : 2, fp4 ? CLPK_DIST_NORMAL : CLPK_DIST_UNIFORM_PM1, 0, 1, w.stream);
            rc |= clpk_memcpy_d2h(dense.data(), f32.p, dense.size() * 4, w.stream);
            rc |= clpk_stream_sync(w.stream);
        }
        if (rc != CLPK_OK)
            return fail(shimError("operand generation"));
        b200check::pruneTile(dense, 128, K, fp4, comp, meta);
        rc |= clpk_memcpy_h2d(f32.p, comp.data(), comp.size() * 4, w.stream);
        rc |= clpk_memcpy_h2d(dMeta.p, meta.data(), meta.size(), w.stream);
        if (fp4)
            rc |= clpk_quantize_fp4(dA.as<uint8_t>(), dSfa.as<uint8_t>(), f32.as<float>(), 128, K / 2,
                                    kind == CLPK_MMA_MXF4_SP ? CLPK_DT_MXF4 : CLPK_DT_NVF4,
                                    kind == CLPK_MMA_MXF4_SP ? 1.0f : 0.001953125f, w.stream);
        else
            rc |= clpk_convert_f32(dA.p, f32.as<float>(), comp.size(), kind == CLPK_MMA_I8_SP ? CLPK_DT_I8 : CLPK_DT_E4M3, w.stream);
        // B: dense
        if (kind == CLPK_MMA_I8_SP)
            rc |= clpk_fill_i8(dB.as<int8_t>(), 256 * (uint64_t)K, 3, w.stream);
        else if (!fp4) {
            rc |= clpk_fill_f32(f32.as<float>(), 256 * (uint64_t)K, 3, CLPK_DIST_UNIFORM_PM1, 0, 1, w.stream);
            rc |= clpk_convert_f32(dB.p, f32.as<float>(), 256 * (uint64_t)K, CLPK_DT_E4M3, w.stream);
        } else {
            rc |= clpk_fill_f32(f32.as<float>(), 256 * (uint64_t)K, 4, CLPK_DIST_NORMAL, 0, 1, w.stream);
            rc |= clpk_quantize_fp4(dB.as<uint8_t>(), dSfb.as<uint8_t>(), f32.as<float>(), 256, K,
                                    kind == CLPK_MMA_MXF4_SP ? CLPK_DT_MXF4_B64 : CLPK_DT_NVF4_B32,
                                    kind == CLPK_MMA_MXF4_SP ? 1.0f : 0.001953125f, w.stream);
        }
        if (rc != CLPK_OK)
            return fail(shimError("operand generation"));

        clpk_mma_peak_args_t a{};
        a.kind = kind;
        a.d_a = dA.p; a.d_b = dB.p; a.d_sfa = dSfa.p; a.d_sfb = dSfb.p; a.d_meta = dMeta.p;
        a.n_mma = nMma; a.grid = grid; a.n_out_tiles = 1;
        a.d_out = dOut.p; a.d_checksum = dChk.as<uint32_t>(); a.d_status = dStatus.as<uint32_t>();
        a.d_clock = dClock.as<unsigned long long>();
        clpk_memset(dClock.p, 0, 16, w.stream);

        std::string err;
        const double s = w.timeLaunches([&] { return clpk_mma_peak(&a, w.stream); }, err);
        if (s < 0)
            return fail(err);

        std::vector<uint8_t> hA(aBytes), hB(bBytes), hSfa(128 * (size_t)nsf), hSfb(256 * (size_t)nsf);
        std::vector<uint32_t> tile(128 * 256), chk(grid);
        uint32_t status = 0;
        unsigned long long clock[2] = {0, 0};
        clpk_memcpy_d2h(clock, dClock.p, sizeof clock, w.stream);
        clpk_memcpy_d2h(hA.data(), dA.p, aBytes, w.stream);
        clpk_memcpy_d2h(hB.data(), dB.p, bBytes, w.stream);
        clpk_memcpy_d2h(hSfa.data(), dSfa.p, hSfa.size(), w.stream);
        clpk_memcpy_d2h(hSfb.data(), dSfb.p, hSfb.size(), w.stream);
        clpk_memcpy_d2h(tile.data(), dOut.p, tile.size() * 4, w.stream);
        clpk_memcpy_d2h(chk.data(), dChk.p, chk.size() * 4, w.stream);
        clpk_memcpy_d2h(&status, dStatus.p, 4, w.stream);
        if (clpk_stream_sync(w.stream) != CLPK_OK)
            return fail(shimError("read back"));
        if (status != 0)
            return fail("a device-side wait timed out (status " + std::to_string(status) + ")");
        for (uint32_t c : chk)
            if (c != chk[0])
                return fail("CTAs disagree on the accumulator checksum");
        double worst = 0;
        const std::string verdict = b200check::checkSparseTile(kind, hA.data(), meta.data(), hB.data(), hSfa.data(), hSfb.data(),
                                                               nMma, tile.data(), &worst);
        if (!verdict.empty())
            return fail("accumulator check failed: " + verdict);

        const double work = clpk_mma_flops_per_instr(kind) * nMma * grid;
        const double t = work / s / 1e12;
        out.readings.push_back(ok(row.metric, t, note + "  " + pct(t, row.spec, row.specName) +
                                                     cyclesNote(s, clock, (double)nMma * grid / w.info.numSMs), work, s));
    }

    // fp64 tensor cores: no tcgen05 kind exists, so this is the warp-level DMMA path (mma.sync.m8n8k4.f64),
    // the successor of wmma_fp64 (src/cuda/wmma.cpp:131-138).  Operands are multiples of 2^-8 so that the
    // expected accumulators are exact in fp64 whatever order the hardware adds the four products in.
    static void tensorFp64(B200Worker &w, B200TestResult &out)
    {
        out.spec = {"wmma_fp64", "DMMA fp64xfp64+fp64 8x8x4", "tflops", Category::Unknown,
                    "Tensor cores on full 64-bit numbers, for scientific computing.  Blackwell's tcgen05 instructions "
                    "have no 64-bit form, so this is the warp-level instruction the earlier generations introduced."};
        const uint32_t grid = 8u * (uint32_t)w.info.numSMs, nMma = 1u << 13;
        const std::string note = "2^13 dependent instructions on each of " + std::to_string(CLPK_DMMA_CHAINS) +
                                 " accumulators per warp, " + std::to_string(CLPK_DMMA_WARPS) + " warps on each of " +
                                 std::to_string(grid) + " CTAs; seeded operands (multiples of 2^-8 in [-1,1)), "
                                 "accumulators compared exactly with the host.";
        auto fail = [&](const std::string &why) { out.readings.push_back(bad("wmma_fp64", ResultStatus::Error, why, note)); };
        double hA[32], hB[32];
        for (int i = 0; i < 32; ++i) {
            hA[i] = std::floor((double)clpk_uniform_pm1(2, (uint64_t)i) * 256.0) / 256.0;
            hB[i] = std::floor((double)clpk_uniform_pm1(2, 32 + (uint64_t)i) * 256.0) / 256.0;
        }
        const uint32_t outTiles = 2;
        DeviceBuffer dA, dB, dOut, dChk;
        if (!dA.alloc(sizeof hA) || !dB.alloc(sizeof hB) || !dOut.alloc(outTiles * CLPK_DMMA_WARPS * 64 * sizeof(double)) ||
            !dChk.alloc(grid * 4))
            return fail("Failed to allocate buffers");
        if (clpk_memcpy_h2d(dA.p, hA, sizeof hA, w.stream) != CLPK_OK || clpk_memcpy_h2d(dB.p, hB, sizeof hB, w.stream) != CLPK_OK)
            return fail(shimError("operand upload"));
        std::string err;
        const double s = w.timeLaunches([&] {
            return clpk_dmma_peak(dA.as<double>(), dB.as<double>(), nMma, grid, outTiles, dOut.as<double>(),
                                  dChk.as<uint32_t>(), w.stream);
        }, err);
        if (s < 0)
            return fail(err);
        std::vector<double> tiles((size_t)outTiles * CLPK_DMMA_WARPS * 64);
        std::vector<uint32_t> chk(grid);
        clpk_memcpy_d2h(tiles.data(), dOut.p, tiles.size() * sizeof(double), w.stream);
        clpk_memcpy_d2h(chk.data(), dChk.p, chk.size() * 4, w.stream);
        if (clpk_stream_sync(w.stream) != CLPK_OK)
            return fail(shimError("read back"));
        for (uint32_t c : chk)
            if (c != chk[0])
                return fail("CTAs disagree on the accumulator checksum");
        for (uint32_t t = 0; t < outTiles; ++t)
            for (int wp = 0; wp < CLPK_DMMA_WARPS; ++wp)
                for (int r = 0; r < 8; ++r)
                    for (int c = 0; c < 8; ++c) {
                        double want = b200check::dmmaExpected(hA, hB, nMma, wp, r, c);
                        const double got = tiles[((size_t)t * CLPK_DMMA_WARPS + wp) * 64 + r * 8 + c];
                        if (got != want)
                            return fail("accumulator check failed: warp " + std::to_string(wp) + " (" + std::to_string(r) + "," +
                                        std::to_string(c) + ") = " + std::to_string(got) + ", host " + std::to_string(want));
                    }
        const double work = 512.0 * nMma * CLPK_DMMA_CHAINS * CLPK_DMMA_WARPS * grid;
        const double t = work / s / 1e12;
        out.readings.push_back(ok("wmma_fp64", t, note + "  " + pct(t, kSpecFp64Tflops, "fp64 tensor TFLOPS"), work, s));
    }

    static void tensorNotBuilt(B200TestResult &out, const char *tag, const char *display, const char *metric,
                               const char *unit, const char *why)
    {
        out.spec = {tag, display, unit, Category::Unknown, ""};
        out.readings.push_back(bad(metric, ResultStatus::Unsupported, why));
    }

    // ---- GEMM -----------------------------------------------------------------------------------

    static uint32_t gemmDim(const B200Worker &w)
    {
        // the reference's sizing (src/cuda/cuda_blas.cpp:132-146): 2048 + 256 per SM, clamped to [2048, 16384]
        // and to a quarter of VRAM for three 2-byte matrices, then rounded to this kernel's 256 tiles.
        uint64_t d = 2048ull + (uint64_t)w.info.numSMs * 256ull;
        d = std::min<uint64_t>(std::max<uint64_t>(d, 2048), 16384);
        while (d > 2048 && 3ull * d * d * 2ull > w.info.totalGlobalMem / 4)
            d -= 256;
        return (uint32_t)(d / 256 * 256);
    }

    struct GemmRow { const char *metric; int dtype; double spec; const char *specName; const char *desc; };

    // One square GEMM row: operands generated and quantised on the device, timed, 16 sampled
    // elements of C compared with a host dot product of the same quantised operands.
    static void gemmRow(B200Worker &w, B200TestResult &out, const GemmRow &r)
    {
        const uint32_t d = gemmDim(w);
        const int dt = r.dtype;
        const bool nv = dt == CLPK_DT_NVF4, mx = dt == CLPK_DT_MXF4, scaled = nv || mx;
        const bool wideOut = dt == CLPK_DT_TF32 || dt == CLPK_DT_I8 || dt == CLPK_DT_F32;
        const uint32_t sfBlock = nv ? 16 : 32;
        const char *outName = dt == CLPK_DT_TF32 ? "fp32 out" : dt == CLPK_DT_I8 ? "int32 accumulate and out"
                            : dt == CLPK_DT_F32 ? "fp32 throughout, on the CUDA cores (FFMA)"
                            : dt == CLPK_DT_F64 ? "fp64 throughout, on the warp-level DMMA instruction" : "fp32 accumulate, bf16 out";
        const std::string note = "M=N=K=" + std::to_string(d) + ", A row-major, B column-major, " +
                                 (dt == CLPK_DT_I8 ? "uniform[-8,7] operands, " : "N(0,0.02) operands, ") +
                                 (nv ? "e2m1 with ue4m3 block scales and fp32 tensor scales (put in tile order once, before timing), " : "") +
                                 (mx ? "e2m1 with ue8m0 block scales (put in tile order once, before timing), " : "") +
                                 (dt == CLPK_DT_E5M2 ? "e5m2 A times e4m3 B, " : "") + outName +
                                 "; sampled elements checked against a host dot product.";
        auto fail = [&](const std::string &why) { out.readings.push_back(bad(r.metric, ResultStatus::Error, why, note)); };
        const uint64_t n = (uint64_t)d * d;
        const uint64_t rowBytes = scaled ? d / 2 : dt == CLPK_DT_F64 ? 8ull * d : (dt == CLPK_DT_TF32 || dt == CLPK_DT_F32) ? 4ull * d
                                : (dt == CLPK_DT_F16 || dt == CLPK_DT_BF16) ? 2ull * d : d;
        const uint64_t outBytes = dt == CLPK_DT_F64 ? 8 : wideOut ? 4 : 2;
        // N(0, 0.02): |x| < 0.12, so a tensor scale of 2^-15 keeps x / scale / 6 within ue4m3's range (448).
        const float tensorScale = nv ? std::ldexp(1.0f, -15) : 1.0f;
        size_t wsBytes = 0;
        if (scaled && clpk_gemm_workspace_bytes(dt, d, d, d, &wsBytes) != CLPK_OK)
            return fail(shimError("workspace size"));
        DeviceBuffer tmp, A, B, C, st, sfa, sfb, ws;
        if (!tmp.alloc(n * 4) || !A.alloc(d * rowBytes) || !B.alloc(d * rowBytes) || !C.alloc(n * outBytes) || !st.alloc(4) ||
            (scaled && (!sfa.alloc(n / sfBlock) || !sfb.alloc(n / sfBlock) || !ws.alloc(wsBytes))))
            return fail("Failed to allocate matrices");
        auto operand = [&](DeviceBuffer &dst, DeviceBuffer &sf, uint64_t seed, bool isB) {
            if (dt == CLPK_DT_I8)
                return clpk_fill_i8(dst.as<int8_t>(), n, seed, w.stream);
            int rc = clpk_fill_f32(tmp.as<float>(), n, seed, CLPK_DIST_NORMAL, 0.0f, 0.02f, w.stream);
            if (scaled)
                return rc | clpk_quantize_fp4(dst.as<uint8_t>(), sf.as<uint8_t>(), tmp.as<float>(), d, d, dt, tensorScale, w.stream);
            if (dt == CLPK_DT_F32)
                return rc | clpk_memcpy_d2d(dst.p, tmp.p, n * 4, w.stream);
            return rc | clpk_convert_f32(dst.p, tmp.as<float>(), n, (dt == CLPK_DT_E5M2 && isB) ? CLPK_DT_E4M3 : dt, w.stream);
        };
        int rc = operand(A, sfa, 40, false);
        rc |= operand(B, sfb, 41, true);
        clpk_gemm_args_t g{};
        g.dtype = dt; g.m = g.n = g.k = d;
        g.d_a = A.p; g.d_b = B.p; g.d_c = C.p; g.d_status = st.as<uint32_t>();
        g.alpha = nv ? tensorScale * tensorScale : 1.0f;
        g.d_sfa = sfa.p; g.d_sfb = sfb.p; g.d_workspace = ws.p; g.workspace_bytes = wsBytes;
        // The scale arrays go into tile order once, as cuBLASLt's caller has to hand them over
        // (src/cuda/cuda_blas.cpp:456-491 prepares them before its timed loop); the timed calls
        // then take the packed workspace as it is.
        if (scaled && rc == CLPK_OK) {
            rc = clpk_gemm_pack_scales(&g, w.stream);
            g.d_sfa = nullptr;
            g.d_sfb = nullptr;
        }
        std::string err;
        const double s = rc == CLPK_OK ? w.timeLaunches([&] { return clpk_gemm(&g, w.stream); }, err) : -1.0;
        if (s < 0)
            return fail(err.empty() ? shimError("operand generation") : err);
        std::string verdict;
        uint32_t status = 0;
        clpk_memcpy_d2h(&status, st.p, 4, w.stream);
        const uint64_t sfRow = d / sfBlock;
        std::vector<uint8_t> rowA(rowBytes), rowB(rowBytes), rowSfa(sfRow), rowSfb(sfRow);
        for (int sidx = 0; sidx < 16 && verdict.empty(); ++sidx) {
            const uint64_t i = clpk_rand64(77, 2 * sidx) % d, j = clpk_rand64(77, 2 * sidx + 1) % d;
            uint32_t cWord = 0;
            double cDouble = 0;
            clpk_memcpy_d2h(rowA.data(), A.as<uint8_t>() + i * rowBytes, rowBytes, w.stream);
            clpk_memcpy_d2h(rowB.data(), B.as<uint8_t>() + j * rowBytes, rowBytes, w.stream);
            if (scaled) {
                clpk_memcpy_d2h(rowSfa.data(), sfa.as<uint8_t>() + i * sfRow, sfRow, w.stream);
                clpk_memcpy_d2h(rowSfb.data(), sfb.as<uint8_t>() + j * sfRow, sfRow, w.stream);
            }
            if (dt == CLPK_DT_F64)
                clpk_memcpy_d2h(&cDouble, C.as<double>() + i * d + j, 8, w.stream);
            else if (wideOut)
                clpk_memcpy_d2h(&cWord, C.as<uint32_t>() + i * d + j, 4, w.stream);
            else
                clpk_memcpy_d2h(&cWord, C.as<uint16_t>() + i * d + j, 2, w.stream);
            clpk_stream_sync(w.stream);
            double sAbs = 0;
            const double want = (double)g.alpha * b200check::gemmElement(dt, rowA.data(), rowB.data(), d, 0, 0, &sAbs,
                                                                         rowSfa.data(), rowSfb.data());
            sAbs *= g.alpha;
            double got, tol;
            if (dt == CLPK_DT_I8) {
                got = (double)(int32_t)cWord;
                tol = 0.0;
            } else if (dt == CLPK_DT_F64) {
                got = cDouble;
                tol = d * std::ldexp(1.0, -51) * sAbs + 1e-300;      // K fp64 roundings on each side of the comparison
            } else if (dt == CLPK_DT_TF32 || dt == CLPK_DT_F32) {
                got = clpk_bits_f32(cWord);
                tol = d * std::ldexp(1.0, -23) * sAbs + 1e-30;
            } else {
                got = clpk_bf16_decode((uint16_t)cWord);
                tol = d * std::ldexp(1.0, -23) * sAbs + std::ldexp(1.0, -8) * std::fabs(want) + 1e-30;
            }
            if (!(std::fabs(got - want) <= tol))
                verdict = "C(" + std::to_string(i) + "," + std::to_string(j) + ") = " + std::to_string(got) +
                          ", host " + std::to_string(want);
        }
        if (status != 0)
            verdict = "a device-side wait timed out (status " + std::to_string(status) + ")";
        if (!verdict.empty())
            return fail("result check failed: " + verdict);
        const double work = 2.0 * d * d * d;
        const double t = work / s / 1e12;
        std::string clockNote;
        unsigned long long cyc = 0, ns = 0;
        if (dt != CLPK_DT_F32 && dt != CLPK_DT_F64 && clpk_gemm_last_clock(&cyc, &ns, w.stream) == CLPK_OK && ns > 0)
            clockNote = "  SM clock inside the last launch: " + std::to_string((long long)((double)cyc / (double)ns * 1e3 + 0.5)) + " MHz.";
        out.readings.push_back(ok(r.metric, t, note + "  " + pct(t, r.spec, r.specName) + clockNote, work, s));
    }

    static void gemmFp(B200Worker &w, B200TestResult &out)
    {
        out.spec = {"cublas-fp", "GEMM peak (in-house tcgen05 GEMM)", "tflops", Category::Unknown,
                    "A whole matrix multiplication C = A*B on the tensor cores, operands streamed from memory by TMA: "
                    "what a well-tuned library routine reaches, as opposed to the bare instruction rate of the rows above.  "
                    "The reference calls cuBLASLt here; this backend runs its own warp-specialised 2-CTA tcgen05 kernel."};
        // the reference's row order (src/cuda/cuda_blas.cpp:567-676)
        static const GemmRow rows[] = {
            {"fp32", CLPK_DT_F32, kSpecFp32Gflops / 1000.0, "fp32 TFLOPS (CUDA cores)", ""},
            {"fp64", CLPK_DT_F64, kSpecFp64Tflops, "fp64 tensor TFLOPS", ""},
            {"tf32", CLPK_DT_TF32, kSpecBf16Tflops / 2, "dense tf32 TFLOPS", ""},
            {"fp16", CLPK_DT_F16, kSpecBf16Tflops, "dense fp16 TFLOPS", ""},
            {"bf16", CLPK_DT_BF16, kSpecBf16Tflops, "dense bf16 TFLOPS", ""},
            {"fp8_e4m3", CLPK_DT_E4M3, kSpecFp8Tflops, "dense fp8 TFLOPS", ""},
            {"fp8_e5m2", CLPK_DT_E5M2, kSpecFp8Tflops, "dense fp8 TFLOPS", ""},
            {"mxf4_e2m1", CLPK_DT_MXF4, kSpecFp4Tflops, "dense fp4 TFLOPS", ""},
            {"nvf4_e2m1", CLPK_DT_NVF4, kSpecFp4Tflops, "dense fp4 TFLOPS", ""},
        };
        for (const GemmRow &r : rows)
            gemmRow(w, out, r);
    }

    static void gemmInt(B200Worker &w, B200TestResult &out)
    {
        out.spec = {"cublas-int", "GEMM peak, integer (in-house tcgen05 GEMM)", "tops", Category::Unknown,
                    "The same matrix multiply on whole-number formats, which is how a quantized (compressed) model actually runs."};
        static const GemmRow int8Row = {"int8", CLPK_DT_I8, kSpecInt8Tops, "dense int8 TOPS", ""};
        gemmRow(w, out, int8Row);
        out.readings.push_back(bad("int4", ResultStatus::Unsupported, "no int4 tensor-core path on sm_100"));
    }

    // ---- bandwidth ------------------------------------------------------------------------------------

    static void globalBandwidth(B200Worker &w, B200TestResult &out)
    {
        out.spec = {"global_memory_bandwidth", "Global memory bandwidth", "gbps", Category::Unknown,
                    "How many bytes per second the GPU can stream out of its own memory, reading a buffer far too "
                    "large to cache.  float/float2/float4 are clpeak's read-and-sum kernels; read, copy and triad "
                    "are STREAM passes over 8 GiB arrays with 128-bit loads or TMA bulk copies."};
        // --- reference read-and-sum rows: 512 MiB (benchmark_config_t::globalBWMaxSize) --------------
        // --- STREAM rows: 8 GiB per array, or what fits in a fifth of VRAM ---------------------------------
        uint64_t streamBytes = 8ull << 30;
        while (streamBytes > (64ull << 20) && 3 * streamBytes > w.info.totalGlobalMem * 3 / 5)
            streamBytes >>= 1;
        const uint64_t nF = streamBytes / 4;
        // whole blocks of the widest variant: 256 threads x 16 fetches x 4 floats
        const uint64_t refFloats = std::min<uint64_t>((1ull << 29) / sizeof(float), nF) / 16384 * 16384;
        DeviceBuffer a, b, c, parts;
        const int variants[3] = {CLPK_STREAM_LDG, CLPK_STREAM_TMA, CLPK_STREAM_WIDE};
        const char *variantName[3] = {"128-bit loads, persistent grid", "TMA bulk copy", "256-bit loads, one 8 KiB tile per CTA"};
        int grids[3] = {0, 0, 0};
        for (int v : variants)
            clpk_stream_read_grid(v, &grids[v]);
        const int grid0 = grids[CLPK_STREAM_LDG];
        const int gridMax = std::max(grids[0], std::max(grids[1], grids[2]));
        if (!a.alloc(streamBytes) || !b.alloc(streamBytes) || !c.alloc(streamBytes) || !parts.alloc((size_t)gridMax * 4)) {
            for (const char *m : {"float", "float2", "float4", "read", "copy", "triad"})
                out.readings.push_back(bad(m, ResultStatus::Error, "Failed to allocate buffers"));
            return;
        }
        clpk_fill_f32(b.as<float>(), nF, 1, CLPK_DIST_UNIFORM01, 0, 1, w.stream);
        clpk_fill_f32(c.as<float>(), nF, 2, CLPK_DIST_UNIFORM01, 0, 1, w.stream);

        const uint64_t headFloats = std::min<uint64_t>(nF, (16ull << 20) / 4);      // 16 MiB checked on the host
        std::vector<float> hb(headFloats), hc(headFloats), ha(headFloats);
        clpk_memcpy_d2h(hb.data(), b.p, headFloats * 4, w.stream);
        clpk_memcpy_d2h(hc.data(), c.p, headFloats * 4, w.stream);
        clpk_stream_sync(w.stream);

        const char *widthNote[3] = {"One value per thread at a time -- the plain, unvectorised case.",
                                    "Two values per thread at a time, packed into one instruction.",
                                    "Four values per thread at a time, as one 4-wide vector."};
        const char *labels[3] = {"float", "float2", "float4"};
        for (int vi = 0; vi < 3; ++vi) {
            const int width = 1 << vi;
            std::string err;
            const double s = w.timeLaunches([&] { return clpk_global_bandwidth(width, b.as<float>(), a.as<float>(), refFloats, w.stream); }, err);
            if (s < 0) {
                out.readings.push_back(bad(labels[vi], ResultStatus::Error, err, widthNote[vi]));
                continue;
            }
            std::vector<float> got(1024);
            clpk_memcpy_d2h(got.data(), a.p, got.size() * 4, w.stream);
            clpk_stream_sync(w.stream);
            bool same = true;
            for (size_t i = 0; i < got.size() && same; ++i)
                same = b200check::sameFloat(got[i], b200check::readSumReference(hb.data(), width, i));
            const double bytes = (double)refFloats * 4;
            if (!same)
                out.readings.push_back(bad(labels[vi], ResultStatus::Error, "sums differ from the host replay", widthNote[vi]));
            else
                out.readings.push_back(ok(labels[vi], bytes / s / 1e9, widthNote[vi], bytes, s));
        }

        auto best = [&](const char *metric, double bytes, const std::function<int(int)> &launch,
                        const std::function<std::string()> &check, const char *what) {
            double bestS = -1;
            int bestV = 0;
            std::string err;
            for (int v : variants) {
                const double s = w.timeLaunches([&] { return launch(v); }, err);
                uint32_t st = 0;
                if (clpk_stream_status(&st, w.stream) != CLPK_OK) {
                    out.readings.push_back(bad(metric, ResultStatus::Error, clpk_last_error(), what));
                    return;
                }
                if (s > 0 && (bestS < 0 || s < bestS)) {
                    bestS = s;
                    bestV = v;
                }
            }
            if (bestS < 0) {
                out.readings.push_back(bad(metric, ResultStatus::Error, err, what));
                return;
            }
            launch(bestV);
            const std::string verdict = check();
            if (!verdict.empty()) {
                out.readings.push_back(bad(metric, ResultStatus::Error, "result check failed: " + verdict, what));
                return;
            }
            const double g = bytes / bestS / 1e9;
            out.readings.push_back(ok(metric, g, std::string(what) + "  Fastest flavour: " + variantName[bestV] +
                                                     ".  " + pct(g, kSpecHbmGBps, "HBM3e GB/s"), bytes, bestS));
        };

        const std::string sz = std::to_string(streamBytes >> 20) + " MiB arrays.";
        best("read", (double)streamBytes,
             [&](int v) { return clpk_stream_read(v, b.p, streamBytes, parts.as<uint32_t>(), w.stream); },
             [&]() -> std::string {
                 // all flavours must agree on the XOR of the whole array, and the head must match the host
                 uint32_t x[3] = {0, 0, 0};
                 for (int v : variants) {
                     std::vector<uint32_t> p((size_t)grids[v]);
                     clpk_stream_read(v, b.p, streamBytes, parts.as<uint32_t>(), w.stream);
                     clpk_memcpy_d2h(p.data(), parts.p, p.size() * 4, w.stream);
                     clpk_stream_sync(w.stream);
                     for (uint32_t q : p) x[v] ^= q;
                 }
                 if (x[0] != x[1] || x[0] != x[2]) return "the flavours disagree on the checksum";
                 std::vector<uint32_t> p((size_t)grid0);
                 clpk_stream_read(CLPK_STREAM_LDG, b.p, headFloats * 4, parts.as<uint32_t>(), w.stream);
                 clpk_memcpy_d2h(p.data(), parts.p, p.size() * 4, w.stream);
                 clpk_stream_sync(w.stream);
                 uint32_t h = 0;
                 for (uint32_t q : p) h ^= q;
                 return h == b200check::xorWords(hb.data(), headFloats * 4) ? "" : "checksum differs from the host";
             },
             ("Reading one large array straight through; XOR checksum of every word verified.  " + sz).c_str());
        best("copy", 2.0 * streamBytes,
             [&](int v) { return clpk_stream_copy(v, a.p, c.p, streamBytes, w.stream); },
             [&]() -> std::string {
                 // XOR(dst) must equal XOR(src) over the whole array; the head must match bit for bit
                 uint32_t x[2] = {0, 0};
                 const void *src[2] = {a.p, c.p};
                 for (int k = 0; k < 2; ++k) {
                     std::vector<uint32_t> p((size_t)grid0);
                     clpk_stream_read(CLPK_STREAM_LDG, src[k], streamBytes, parts.as<uint32_t>(), w.stream);
                     clpk_memcpy_d2h(p.data(), parts.p, p.size() * 4, w.stream);
                     clpk_stream_sync(w.stream);
                     for (uint32_t q : p) x[k] ^= q;
                 }
                 if (x[0] != x[1]) return "checksum of the copy differs from the source";
                 clpk_memcpy_d2h(ha.data(), a.p, headFloats * 4, w.stream);
                 clpk_stream_sync(w.stream);
                 return std::memcmp(ha.data(), hc.data(), headFloats * 4) == 0 ? "" : "head of the copy differs";
             },
             ("Copying one large array into another -- a read and a write for every element.  " + sz).c_str());
        best("triad", 3.0 * streamBytes,
             [&](int v) { return clpk_stream_triad(v, a.as<float>(), b.as<float>(), c.as<float>(), 1.5f, nF, w.stream); },
             [&]() -> std::string {
                 clpk_memcpy_d2h(ha.data(), a.p, headFloats * 4, w.stream);
                 clpk_stream_sync(w.stream);
                 for (uint64_t i = 0; i < headFloats; ++i) {
                     const float t = 1.5f * hc[i];
                     const float want = hb[i] + t;
                     if (!b200check::sameFloat(ha[i], want)) return "element " + std::to_string(i) + " differs from the host";
                 }
                 return "";
             },
             ("Scaling one array, adding a second and storing to a third: two reads and a write per element.  " + sz).c_str());
    }

    static void localBandwidth(B200Worker &w, B200TestResult &out)
    {
        out.spec = {"local_memory_bandwidth", "Local memory bandwidth", "gbps", Category::Unknown,
                    "How many bytes per second the GPU moves through shared memory -- the small on-chip scratchpad a "
                    "block of threads passes data through, which never goes out to the card's main memory."};
        const char *widthNote[3] = {"One value per thread at a time -- the plain, unvectorised case.",
                                    "Two values per thread at a time, packed into one instruction.",
                                    "Four values per thread at a time, as one 4-wide vector."};
        const char *labels[3] = {"float", "float2", "float4"};
        const uint64_t threads = targetGlobalThreads((uint32_t)w.info.numSMs);
        const uint32_t blocks = (uint32_t)(threads / 256);
        DeviceBuffer buf;
        if (!buf.alloc(threads * sizeof(float))) {
            for (int vi = 0; vi < 3; ++vi)
                out.readings.push_back(bad(labels[vi], ResultStatus::Error, "Buffer alloc failed", widthNote[vi]));
            return;
        }
        for (int vi = 0; vi < 3; ++vi) {
            const int width = 1 << vi;
            std::string err;
            const double s = w.timeLaunches([&] { return clpk_local_bandwidth(width, buf.as<float>(), blocks, w.stream); }, err);
            if (s < 0) {
                out.readings.push_back(bad(labels[vi], ResultStatus::Error, err, widthNote[vi]));
                continue;
            }
            // first two blocks and the last one against the closed form
            std::vector<float> head(512), tail(256);
            clpk_memcpy_d2h(head.data(), buf.p, head.size() * 4, w.stream);
            clpk_memcpy_d2h(tail.data(), buf.as<float>() + (threads - 256), tail.size() * 4, w.stream);
            clpk_stream_sync(w.stream);
            bool same = true;
            for (uint64_t i = 0; i < 512 && same; ++i)
                same = b200check::sameFloat(head[i], b200check::localBandwidthReference(width, i));
            for (uint64_t i = 0; i < 256 && same; ++i)
                same = b200check::sameFloat(tail[i], b200check::localBandwidthReference(width, threads - 256 + i));
            const double bytes = (double)LMEM_REPS * 2.0 * width * sizeof(float) * (double)threads;
            if (!same)
                out.readings.push_back(bad(labels[vi], ResultStatus::Error, "outputs differ from the closed form", widthNote[vi]));
            else
                out.readings.push_back(ok(labels[vi], bytes / s / 1e9, widthNote[vi], bytes, s));
        }
    }

    static void imageBandwidth(B200Worker &w, B200TestResult &out)
    {
        out.spec = {"image_memory_bandwidth", "Image memory bandwidth", "gbps", Category::Unknown,
                    "How many bytes per second the GPU reads through its texture units, which take a different path "
                    "to memory than plain buffer reads.  Each pixel of the image is read exactly once, so caching "
                    "cannot flatter the number."};
        const char *note = "Each fetch returns one whole pixel -- four 32-bit colour values, 16 bytes.";
        const uint32_t imgW = 4096, imgH = 4096;
        const uint64_t texels = (uint64_t)imgW * imgH, threads = texels / IMAGE_FETCH_PER_WI;
        const uint32_t blocks = (uint32_t)(threads / 256);
        const uint64_t seed = 5;
        void *image = nullptr;
        if (clpk_image_create(&image, imgW, imgH, seed, w.stream) != CLPK_OK) {
            out.readings.push_back(bad("float4", ResultStatus::Error, shimError("image create"), note));
            return;
        }
        DeviceBuffer buf;
        if (!buf.alloc(threads * sizeof(float))) {
            clpk_image_destroy(image);
            out.readings.push_back(bad("float4", ResultStatus::Error, "Buffer alloc failed", note));
            return;
        }
        std::string err;
        const double s = w.timeLaunches([&] { return clpk_image_bandwidth(image, buf.as<float>(), blocks, w.stream); }, err);
        if (s < 0) {
            out.readings.push_back(bad("float4", ResultStatus::Error, err, note));
        } else {
            std::vector<float> head(256), tail(256);
            clpk_memcpy_d2h(head.data(), buf.p, head.size() * 4, w.stream);
            clpk_memcpy_d2h(tail.data(), buf.as<float>() + (threads - 256), tail.size() * 4, w.stream);
            clpk_stream_sync(w.stream);
            bool same = true;
            for (uint64_t i = 0; i < 256 && same; ++i)
                same = b200check::sameFloat(head[i], b200check::imageBandwidthReference(i, threads, texels, seed)) &&
                       b200check::sameFloat(tail[i], b200check::imageBandwidthReference(threads - 256 + i, threads, texels, seed));
            const double bytes = (double)IMAGE_FETCH_PER_WI * 4.0 * sizeof(float) * (double)threads;
            if (!same)
                out.readings.push_back(bad("float4", ResultStatus::Error, "sums differ from the host replay", note));
            else
                out.readings.push_back(ok("float4", bytes / s / 1e9, note, bytes, s));
        }
        // The same pixels, the same sums per fetch, in an order laid out for the texture path: each
        // block reads 16 neighbouring 8 x 32 pixel tiles instead of 16 row segments 256 rows apart.
        const char *tiledNote = "The same image read in small square-ish patches, the order texture hardware is built "
                                "for (a block of threads reads 16 neighbouring 8 x 32 pixel tiles).";
        const double st = w.timeLaunches([&] { return clpk_image_bandwidth_tiled(image, buf.as<float>(), blocks, w.stream); }, err);
        if (st < 0) {
            out.readings.push_back(bad("float4_tiled", ResultStatus::Error, err, tiledNote));
        } else {
            std::vector<float> head(256), tail(256);
            clpk_memcpy_d2h(head.data(), buf.p, head.size() * 4, w.stream);
            clpk_memcpy_d2h(tail.data(), buf.as<float>() + (threads - 256), tail.size() * 4, w.stream);
            clpk_stream_sync(w.stream);
            bool same = true;
            for (uint64_t i = 0; i < 256 && same; ++i)
                same = b200check::sameFloat(head[i], b200check::imageBandwidthTiledReference(i, imgW, imgH, seed)) &&
                       b200check::sameFloat(tail[i], b200check::imageBandwidthTiledReference(threads - 256 + i, imgW, imgH, seed));
            const double bytes = (double)IMAGE_FETCH_PER_WI * 4.0 * sizeof(float) * (double)threads;
            if (!same)
                out.readings.push_back(bad("float4_tiled", ResultStatus::Error, "sums differ from the host replay", tiledNote));
            else
                out.readings.push_back(ok("float4_tiled", bytes / st / 1e9, tiledNote, bytes, st));
        }
        clpk_image_destroy(image);
    }

    static void transferBandwidth(B200Worker &w, B200TestResult &out)
    {
        out.spec = {"transfer_bandwidth", "Transfer bandwidth", "gbps", Category::Unknown,
                    "How fast data moves between host memory and the GPU over the PCIe link, from page-locked host memory."};
        const char *h2dNote = "Host to device: sending data up to the card.";
        const char *d2hNote = "Device to host: reading results back down.";
        const size_t bytes = 1ull << 29;         // benchmark_config_t::transferBWMaxSize
        DeviceBuffer d;
        PinnedBuffer h;
        if (!d.alloc(bytes) || !h.alloc(bytes)) {
            out.readings.push_back(bad("h2d_pinned", ResultStatus::Error, "Failed to allocate buffers", h2dNote));
            out.readings.push_back(bad("d2h_pinned", ResultStatus::Error, "Failed to allocate buffers", d2hNote));
            return;
        }
        std::memset(h.p, 0x5A, bytes);
        std::string err;
        double s = w.timeLaunches([&] { return clpk_memcpy_h2d(d.p, h.p, bytes, w.stream); }, err);
        out.readings.push_back(s > 0 ? ok("h2d_pinned", bytes / s / 1e9, h2dNote, (double)bytes, s)
                                     : bad("h2d_pinned", ResultStatus::Error, err, h2dNote));
        s = w.timeLaunches([&] { return clpk_memcpy_d2h(h.p, d.p, bytes, w.stream); }, err);
        out.readings.push_back(s > 0 ? ok("d2h_pinned", bytes / s / 1e9, d2hNote, (double)bytes, s)
                                     : bad("d2h_pinned", ResultStatus::Error, err, d2hNote));
    }

    // ---- latency --------------------------------------------------------------------------------------------

    // The chase cycle is identical for every GPU (same seed): build it once per run.
    struct SharedCycle {
        std::mutex m;
        std::vector<uint32_t> next;
        uint64_t n = 0;
        const std::vector<uint32_t> &get(uint64_t want)
        {
            std::lock_guard<std::mutex> lk(m);
            if (n != want) {
                next.assign(want, 0);
                clpk_build_chase_cycle(next.data(), want, 9);
                n = want;
            }
            return next;
        }
    };

    static void memoryLatency(B200Worker &w, B200TestResult &out, SharedCycle &big, SharedCycle &small)
    {
        out.spec = {"memory_latency", "Memory latency (pointer-chase)", "ns", Category::Latency,
                    "How long one dependent load takes: a single thread follows a random cycle of indices, so every "
                    "hop has to wait for the one before it."};
        struct Case { const char *metric; SharedCycle *cycle; uint64_t n, hops; const char *note; };
        const Case cases[] = {
            {"L2", &small, 1ull << 22, 1ull << 20, "16 MiB working set: resident in the L2 cache."},
            {"HBM", &big, 1ull << 28, 1ull << 24, "1 GiB working set (2^28 indices, seeded Sattolo cycle), 2^24 hops: every hop goes to HBM."},
        };
        for (const Case &cs : cases) {
            const std::vector<uint32_t> &next = cs.cycle->get(cs.n);
            DeviceBuffer d, res;
            if (!d.alloc(cs.n * 4) || !res.alloc(16)) {
                out.readings.push_back(bad(cs.metric, ResultStatus::Error, "Failed to allocate buffers", cs.note));
                continue;
            }
            clpk_memcpy_h2d(d.p, next.data(), cs.n * 4, w.stream);
            uint32_t r[4] = {0, 0, 0, 0};
            int rc = clpk_pointer_chase(d.as<uint32_t>(), 0, cs.hops / 16, res.as<uint32_t>(), w.stream);   // warm-up
            rc |= clpk_pointer_chase(d.as<uint32_t>(), 0, cs.hops, res.as<uint32_t>(), w.stream);
            rc |= clpk_memcpy_d2h(r, res.p, 16, w.stream);
            rc |= clpk_stream_sync(w.stream);
            if (rc != CLPK_OK) {
                out.readings.push_back(bad(cs.metric, ResultStatus::Error, shimError("pointer chase"), cs.note));
                continue;
            }
            uint32_t cur = 0, x = 0;
            for (uint64_t h = 0; h < cs.hops; ++h) {
                cur = next[cur];
                x ^= cur;
            }
            if (cur != r[0] || x != r[1]) {
                out.readings.push_back(bad(cs.metric, ResultStatus::Error, "walk differs from the host replay", cs.note));
                continue;
            }
            const double ns = (double)(((uint64_t)r[3] << 32) | r[2]) / (double)cs.hops;
            out.readings.push_back(ok(cs.metric, ns, cs.note));
        }
    }

    static void kernelLatency(B200Worker &w, B200TestResult &out)
    {
        out.spec = {"kernel_launch_latency", "Kernel launch latency", "us", Category::Unknown,
                    "The overhead of asking the GPU to do anything at all, measured with a kernel that does no work."};
        const char *dispatchNote = "One way only: from the moment the host submits the work to the moment the GPU starts "
                                   "running it.  CUDA exposes no clock the host and GPU share, so this is not reported here.";
        const char *roundNote = "The full round trip -- submit, run, and hear back that it finished.";
        out.readings.push_back(bad("dispatch", ResultStatus::Unsupported, "Not measurable via CUDA driver API", dispatchNote));
        double mean = 0;
        if (clpk_launch_latency(w.latencyIters, w.warmup, &mean, w.stream) != CLPK_OK)
            out.readings.push_back(bad("roundtrip", ResultStatus::Error, shimError("launch"), roundNote));
        else
            out.readings.push_back(ok("roundtrip", mean, roundNote));
        // What a launch costs once a launch-bound loop is recorded as a CUDA graph and replayed.
        const char *graphNote = "Per kernel when 1000 empty kernels are recorded once as a CUDA graph and the graph is "
                                "submitted as a whole -- what a launch costs a program that replays its work.";
        const uint32_t graphIters = w.latencyIters > 100 ? w.latencyIters / 100 : 1;
        if (clpk_graph_launch_latency(1000, graphIters, w.warmup, &mean, w.stream) != CLPK_OK)
            out.readings.push_back(bad("graph_node", ResultStatus::Error, shimError("graph launch"), graphNote));
        else
            out.readings.push_back(ok("graph_node", mean, graphNote));
    }
};

// ---------------------------------------------------------------------------------
// CudaPeak
// ---------------------------------------------------------------------------------

CudaPeak::CudaPeak() {}
CudaPeak::~CudaPeak() {}

void CudaPeak::applyOptions(const CliOptions &opts)
{
    Peak::applyOptions(opts);
    deviceIndices = opts.cudaDeviceIndices;
}

static bool queryDevice(int idx, cuda_device_info_t &out)
{
    clpk_device_info_t di;
    if (clpk_device_info(idx, &di) != CLPK_OK)
        return false;
    out.index = idx;
    out.deviceName = di.name;
    out.ccMajor = di.cc_major;
    out.ccMinor = di.cc_minor;
    out.numSMs = di.num_sms;
    out.totalGlobalMem = di.total_mem_bytes;
    out.archName = "sm_" + std::to_string(di.cc_major) + std::to_string(di.cc_minor);
    out.driverVersion = std::to_string(di.driver_version / 1000) + "." + std::to_string((di.driver_version % 1000) / 10);
    out.runtimeVersion = std::to_string(di.runtime_version / 1000) + "." + std::to_string((di.runtime_version % 1000) / 10);
    return true;
}

BackendInventory CudaPeak::enumerate()
{
    BackendInventory inv;
    inv.backend = "CUDA";
    int n = 0;
    if (clpk_device_count(&n) != CLPK_OK || n == 0)
        return inv;
    inv.available = true;
    InventoryPlatform plat;
    plat.index = 0;
    plat.name = "CUDA";
    for (int i = 0; i < n; ++i) {
        cuda_device_info_t di;
        if (!queryDevice(i, di))
            continue;
        InventoryDevice d;
        d.index = i;
        d.name = di.deviceName;
        d.typeStr = di.archName;
        plat.devices.push_back(d);
    }
    inv.platforms.push_back(plat);
    return inv;
}

void CudaPeak::printInventory(const BackendInventory &b, std::ostream &os)
{
    os << "\n=== CUDA backend ===\n";
    if (!b.available) {
        os << "CUDA: driver init failed or no devices found\n";
        return;
    }
    for (const auto &p : b.platforms)
        for (const auto &d : p.devices) {
            os << "  CUDA Device " << d.index << ": " << d.name;
            if (!d.typeStr.empty())
                os << " [" << d.typeStr << "]";
            os << "\n";
        }
}

int CudaPeak::runAll()
{
    int count = 0;
    const int rc = clpk_device_count(&count);
    if (rc == CLPK_ERR_NO_DEVICE || (rc == CLPK_OK && count == 0)) {
        log->note("CUDA: no devices found\n");
        return 0;
    }
    if (rc != CLPK_OK) {
        log->note("CUDA: driver init failed\n");
        return -1;
    }

    // ---- selection --------------------------------------------------------------------------
    std::vector<std::unique_ptr<B200Worker>> workers;
    for (int i = 0; i < count; ++i) {
        if (!deviceIndices.empty() && std::find(deviceIndices.begin(), deviceIndices.end(), i) == deviceIndices.end())
            continue;
        auto w = std::make_unique<B200Worker>();
        w->device = i;
        if (!queryDevice(i, w->info)) {
            log->note("CUDA: failed to init device " + std::to_string(i) + "\n");
            continue;
        }
        if (w->info.ccMajor != 10) {
            log->note("CUDA: device " + std::to_string(i) + " (" + w->info.deviceName + ", " + w->info.archName +
                      ") is not sm_100; this backend has no kernels for it\n");
            continue;
        }
        w->warmup = warmupCount;
        w->targetUs = targetTimeUs;
        w->forcedIters = forceIters ? specifiedIters : 0;
        w->latencyIters = forceIters ? specifiedIters : benchmark_config_t::forDevice(DeviceType::Gpu).kernelLatencyIters;
        workers.push_back(std::move(w));
    }
    if (workers.empty())
        return 0;

    // ---- plan: the reference's phase order (cuda_peak.cpp:165-202) ----------------------------------
    using H = B200Harness;
    auto sharedBig = std::make_shared<H::SharedCycle>();
    auto sharedSmall = std::make_shared<H::SharedCycle>();
    std::vector<H::Test> plan;
    const bool fp = isAllowedAs(Benchmark::Wmma, Category::FpCompute);
    if (isAllowed(Benchmark::ComputeSP))
        plan.push_back(H::computeSP);
    {
        // same order as the reference's floating phase (src/cuda/cuda_peak.cpp:165-174)
        const Benchmark fpChains[] = {Benchmark::ComputeHP, Benchmark::ComputeDP, Benchmark::ComputeMP, Benchmark::ComputeBF16};
        for (size_t i = 0; i < 4; ++i)
            if (isAllowed(fpChains[i])) {
                const H::ChainTest &t = H::chainTests()[i];
                plan.push_back([&t](B200Worker &w, B200TestResult &o) { H::typedChain(w, o, t); });
            }
    }
    if (fp) {
        // the reference's row order (src/cuda/wmma.cpp): fp16, fp16 acc, bf16, tf32, fp64, fp8 x2, fp4, mxf4, nvf4, sparse
        for (const auto &row : H::kindRows()) {
            if (row.kind == CLPK_MMA_I8)
                continue;
            plan.push_back([row](B200Worker &w, B200TestResult &o) { H::tensorPeak(w, o, row); });
            if (row.kind == CLPK_MMA_TF32)
                plan.push_back(H::tensorFp64);
        }
        for (const auto &row : H::sparseRows(false))
            plan.push_back([row](B200Worker &w, B200TestResult &o) { H::tensorSparse(w, o, row); });
    }
    if (isAllowedAs(Benchmark::Cublas, Category::FpCompute))
        plan.push_back(H::gemmFp);
    if (isAllowed(Benchmark::ComputeInt)) {
        const H::ChainTest &t = H::chainTests()[4];
        plan.push_back([&t](B200Worker &w, B200TestResult &o) { H::typedChain(w, o, t); });
    }
    if (isAllowed(Benchmark::ComputeInt8DP)) {
        const H::ChainTest &t = H::chainTests()[5];
        plan.push_back([&t](B200Worker &w, B200TestResult &o) { H::typedChain(w, o, t); });
    }
    if (isAllowedAs(Benchmark::Wmma, Category::IntCompute)) {
        plan.push_back([](B200Worker &, B200TestResult &o) { H::tensorNotBuilt(o, "wmma_int8", "wmma int8 16x16x16", "wmma_int8", "tops", "superseded by the tcgen05 int8_k32 row on sm_100"); });
        for (const auto &row : H::kindRows())
            if (row.kind == CLPK_MMA_I8)
                plan.push_back([row](B200Worker &w, B200TestResult &o) { H::tensorPeak(w, o, row); });
        for (const auto &row : H::sparseRows(true))
            plan.push_back([row](B200Worker &w, B200TestResult &o) { H::tensorSparse(w, o, row); });
        plan.push_back([](B200Worker &, B200TestResult &o) { H::tensorNotBuilt(o, "wmma_int4", "int4 tensor path", "int4", "tops", "no int4 tensor-core path on sm_100"); });
    }
    if (isAllowedAs(Benchmark::Cublas, Category::IntCompute))
        plan.push_back(H::gemmInt);
    if (isAllowed(Benchmark::GlobalBW))
        plan.push_back(H::globalBandwidth);
    if (isAllowed(Benchmark::LocalBW))
        plan.push_back(H::localBandwidth);
    if (isAllowed(Benchmark::ImageBW))
        plan.push_back(H::imageBandwidth);
    if (isAllowed(Benchmark::TransferBW))
        plan.push_back(H::transferBandwidth);
    if (isAllowed(Benchmark::MemoryLatency))
        plan.push_back([sharedBig, sharedSmall](B200Worker &w, B200TestResult &o) { H::memoryLatency(w, o, *sharedBig, *sharedSmall); });
    if (isAllowed(Benchmark::KernelLatency))
        plan.push_back(H::kernelLatency);

    // ---- run: one thread per GPU, start gate before every test ---------------------------------------------
    // Two gates: `gate` lines the threads up at the start of each test (allocation and operand
    // generation take different times per GPU), `batchGate` again right before each timed batch.
    // A thread that errors out of a test early never reaches that test's batch gate; the others
    // give up on it after batchGateTimeout, the gate is marked broken and later batches start
    // unsynchronised (the per-test gate keeps working).
    StartGate gate((int)workers.size()), batchGate((int)workers.size());
    const auto gateTimeout = std::chrono::milliseconds(barrierTimeoutMs);
    std::vector<std::thread> threads;
    for (auto &wp : workers) {
        B200Worker *w = wp.get();
        if (workers.size() > 1) {
            w->batchGate = &batchGate;
            w->batchGateTimeout = std::min(gateTimeout, std::chrono::milliseconds(20000));
        }
        threads.emplace_back([w, &plan, &gate, &batchGate, gateTimeout] {
            bool alive = clpk_set_device(w->device) == CLPK_OK && clpk_stream_create(&w->stream) == CLPK_OK;
            if (!alive)
                w->fatal = shimError("device init");
            for (size_t t = 0; t < plan.size() && alive; ++t) {
                if (clpeak::cancelRequested())
                    break;
                gate.arrive(gateTimeout);
                B200TestResult r;
                try {
                    plan[t](*w, r);
                } catch (const std::exception &e) {
                    r.readings.push_back(B200Harness::bad("(test)", ResultStatus::Error, std::string("exception: ") + e.what()));
                }
                w->push(std::move(r));
            }
            gate.leave();
            batchGate.leave();
            if (w->stream)
                clpk_stream_destroy(w->stream);
            {
                std::lock_guard<std::mutex> lk(w->m);
                w->finished = true;
            }
            w->cv.notify_all();
        });
    }

    // ---- emit: calling thread only ---------------------------------------------------------------------------------
    const bool many = workers.size() > 1;
    auto backendScope = log->beginBackend("CUDA");
    std::vector<std::vector<B200TestResult>> all(workers.size());
    for (size_t wi = 0; wi < workers.size(); ++wi) {
        B200Worker &w = *workers[wi];
        // Several identical GPUs would share one result key and one <run>; the index keeps them apart.
        const std::string name = many ? w.info.deviceName + " #" + std::to_string(w.device) : w.info.deviceName;
        auto deviceScope = backendScope.beginDevice({name, "", w.info.driverVersion,
                                                     {{"Arch", w.info.archName},
                                                      {"Toolkit", w.info.runtimeVersion},
                                                      {"SMs", std::to_string(w.info.numSMs)},
                                                      {"VRAM", std::to_string(w.info.totalGlobalMem / (1024 * 1024)) + " MB"}},
                                                     -1, w.device});
        for (;;) {
            B200TestResult r;
            {
                std::unique_lock<std::mutex> lk(w.m);
                w.cv.wait(lk, [&] { return !w.ready.empty() || w.finished; });
                if (w.ready.empty())
                    break;
                r = std::move(w.ready.front());
                w.ready.pop_front();
            }
            if (!r.spec.tag.empty()) {
                auto test = deviceScope.beginTest(r.spec);
                for (const B200Reading &m : r.readings) {
                    if (m.status == ResultStatus::Ok)
                        test.emit(m.metric, m.value, logger::EmitOptions{false, m.info});
                    else
                        test.skip(m.metric, m.status, m.reason, m.info);
                }
            }
            all[wi].push_back(std::move(r));
        }
        if (!w.fatal.empty())
            log->note("CUDA: device " + std::to_string(w.device) + ": " + w.fatal + "\n");
    }
    for (auto &t : threads)
        t.join();
    if (gate.broken())
        log->note("CUDA: a device thread missed the start gate; the remaining tests ran unsynchronised\n");
    if (batchGate.broken())
        log->note("CUDA: a device thread missed a timed-batch gate; later batches started unsynchronised\n");

    // ---- box aggregate ------------------------------------------------------------------------------------------------
    if (many && !clpeak::cancelRequested()) {
        auto agg = backendScope.beginDevice({workers[0]->info.deviceName + " x" + std::to_string(workers.size()) + " (box aggregate)",
                                             "", workers[0]->info.driverVersion,
                                             {{"GPUs", std::to_string(workers.size())},
                                              {"Aggregation", "sum of work / slowest GPU's time; latencies averaged"}},
                                             -1, -1});
        const size_t nTests = all[0].size();
        for (size_t t = 0; t < nTests; ++t) {
            const B200TestResult &first = all[0][t];
            if (first.spec.tag.empty())
                continue;
            auto test = agg.beginTest(first.spec);
            for (size_t mi = 0; mi < first.readings.size(); ++mi) {
                const B200Reading &m0 = first.readings[mi];
                double work = 0, slow = 0, sum = 0;
                size_t okCount = 0;
                for (size_t wi = 0; wi < all.size(); ++wi) {
                    if (t >= all[wi].size() || mi >= all[wi][t].readings.size())
                        continue;
                    const B200Reading &m = all[wi][t].readings[mi];
                    if (m.status != ResultStatus::Ok)
                        continue;
                    ++okCount;
                    sum += m.value;
                    work += m.work;
                    slow = std::max(slow, m.seconds);
                }
                if (okCount != all.size()) {
                    test.skip(m0.metric, m0.status == ResultStatus::Ok ? ResultStatus::Error : m0.status,
                              m0.status == ResultStatus::Ok ? "not every GPU produced this reading" : m0.reason);
                    continue;
                }
                const bool latency = (first.spec.unit == "us" || first.spec.unit == "ns");
                double v;
                if (latency)
                    v = sum / okCount;
                else if (work > 0 && slow > 0)
                    v = work / slow / (first.spec.unit[0] == 't' ? 1e12 : 1e9);
                else
                    v = sum;
                test.emit(m0.metric, (float)v, logger::EmitOptions{false, latency ? "mean over the GPUs" : "all GPUs running at the same time"});
            }
        }
    }
    return 0;
}
