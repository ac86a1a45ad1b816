// The host-side contract a clpeak backend is written against, restated in one
// header: the test registry (Benchmark / Category), the result row and device
// metadata records, the scoped logger that turns a backend's emit() calls into
// an event stream plus an accumulated result table, the parsed command line,
// and the abstract Peak backend class.
//
// Every public name, signature and default here matches the reference tree, so
// that a backend source file compiles unchanged against either this header or
// the reference's own include/common/*.h (the thin headers under common/ make
// the reference's include paths resolve here):
//   Benchmark, Category, categoryOf     include/common/benchmark_enums.h:17-145
//   ResultEntry, DeviceInfo, save*/load* include/common/result_store.h:13-149
//   logger + scopes, LogEvent            include/common/logger.h:36-285
//   CliOptions, parseCliOptions*         include/common/options.h:13-94
//   Peak                                 include/common/peak.h:12-62
//   tuning constants, pickIters          include/common/common.h:55-219
//   BackendInventory                     include/common/inventory.h
#ifndef CLPEAK_B200_HOST_API_HPP
#define CLPEAK_B200_HOST_API_HPP

#include <algorithm>
#include <bitset>
#include <chrono>
#include <cstdint>
#include <cstdio>
#include <initializer_list>
#include <iosfwd>
#include <iostream>
#include <map>
#include <memory>
#include <string>
#include <vector>

#if defined(__linux__) && defined(__x86_64__)
#define OS_NAME "Linux x64"
#elif defined(__linux__) && defined(__aarch64__)
#define OS_NAME "Linux ARM64"
#elif defined(__linux__)
#define OS_NAME "Linux unknown"
#else
#define OS_NAME "Unknown"
#endif

#ifndef CLPEAK_VERSION_STR
#define CLPEAK_VERSION_STR "2.0.16-b200"
#endif

#define TAB "  "
#define NEWLINE "\n"

// ===========================================================================
// Registry
// ===========================================================================

enum class DeviceType : unsigned int { Cpu = 1u << 0, Gpu = 1u << 1, Accelerator = 1u << 2, Unknown = 0 };

// Same members, same order as the reference: the bit index of a test in
// CliOptions::enabledTests is its enum value.
enum class Benchmark : unsigned int {
    GlobalBW = 0, LocalBW, ImageBW,
    ComputeHP, ComputeMP, ComputeSP, ComputeDP,
    ComputeInt, ComputeIntFast, ComputeChar, ComputeShort,
    ComputeInt8DP, ComputeInt16DP, ComputeBF16, ComputeFP8DP, ComputeDivSqrt, ComputeIntDiv,
    CoopMatrix, Wmma, SimdgroupMatrix, MpsGemm, MpsAttention, Cublas,
    Rocwmma, Mfma, Rocblas, JointMatrix, Onemkl, Amx, AppleBlas,
    CryptoAes, CryptoSha256, CryptoSha512, CryptoCrc32c,
    StringScan, Utf8Validate, TextureSample,
    TransferBW, CacheBandwidth, MemoryLatency, Atomics, BranchPenalty, StoreForward, SmtScaling,
    KernelLatency,
    COUNT
};

enum class Category { FpCompute, IntCompute, Crypto, String, Bandwidth, Latency, Unknown };

// Primary category of a test.  Tensor and vendor-library tests (Wmma, Cublas,
// ...) are filed under fp_compute and visited a second time in the integer
// phase through Peak::isAllowedAs.
inline Category categoryOf(Benchmark b)
{
    using B = Benchmark;
    switch (b) {
    case B::GlobalBW: case B::LocalBW: case B::ImageBW: case B::TransferBW:
    case B::CacheBandwidth: case B::TextureSample:
        return Category::Bandwidth;
    case B::ComputeSP: case B::ComputeHP: case B::ComputeDP: case B::ComputeMP: case B::ComputeBF16:
    case B::ComputeFP8DP: case B::ComputeDivSqrt: case B::Wmma: case B::CoopMatrix:
    case B::SimdgroupMatrix: case B::Cublas: case B::MpsGemm: case B::MpsAttention: case B::Rocwmma:
    case B::Mfma: case B::Rocblas: case B::JointMatrix: case B::Onemkl: case B::Amx: case B::AppleBlas:
    case B::SmtScaling:
        return Category::FpCompute;
    case B::ComputeInt: case B::ComputeIntFast: case B::ComputeChar: case B::ComputeShort:
    case B::ComputeInt8DP: case B::ComputeInt16DP: case B::ComputeIntDiv:
        return Category::IntCompute;
    case B::CryptoAes: case B::CryptoSha256: case B::CryptoSha512: case B::CryptoCrc32c:
        return Category::Crypto;
    case B::StringScan: case B::Utf8Validate:
        return Category::String;
    case B::KernelLatency: case B::MemoryLatency: case B::Atomics: case B::BranchPenalty:
    case B::StoreForward:
        return Category::Latency;
    case B::COUNT:
        break;
    }
    return Category::Unknown;
}

// ===========================================================================
// Tuning constants and small helpers
// ===========================================================================

static const unsigned int FETCH_PER_WI = 16;
static const unsigned int LMEM_REPS = 64;
static const unsigned int IMAGE_FETCH_PER_WI = 16;
static const unsigned int COMPUTE_FP_WORK_PER_WI = 4096;
static const unsigned int COMPUTE_DP_WORK_PER_WI = 512;
static const unsigned int COMPUTE_INT_WORK_PER_WI = 2048;
static const unsigned int COMPUTE_INT8_DP_WORK_PER_WI = 8192;
static const unsigned int COOPMAT_WORK_PER_WI = 65536;
static const unsigned int MAX_WG_SIZE = 256;
static const unsigned int DEFAULT_TARGET_TIME_US = 500000;
static const unsigned int DEFAULT_CPU_TARGET_TIME_US = 2000000;

// Threads per launch for the shader-core tests: 2048 work-groups of 256 per
// compute unit, never fewer than 32 Mi.
static inline uint64_t targetGlobalThreads(uint32_t numCUs)
{
    return std::max<uint64_t>(32ull << 20, (uint64_t)numCUs * 2048ull * MAX_WG_SIZE);
}

// Iterations that fill `target_us` given one measured iteration (0 => 5 s),
// clamped to [1, max_iters]; `forced` (non-zero) wins.
unsigned int pickIters(double per_iter_us, unsigned int target_us, unsigned int forced,
                       unsigned int max_iters = 10000);

void populate(float *ptr, uint64_t N);
std::string jsonEscape(const std::string &s);

struct benchmark_config_t {
    uint64_t globalBWMaxSize;
    unsigned int computeWgsPerCU;
    unsigned int computeDPWgsPerCU;
    unsigned int targetTimeUs;
    unsigned int kernelLatencyIters;
    uint64_t transferBWMaxSize;
    static benchmark_config_t forDevice(DeviceType type);
};

namespace clpeak {
bool verboseEnabled();
void setVerbose(bool on);
void requestCancel();
bool cancelRequested();
void resetCancel();
} // namespace clpeak

#define CLPEAK_VLOG(...)                              \
    do {                                              \
        if (::clpeak::verboseEnabled())               \
            fprintf(stderr, __VA_ARGS__);             \
    } while (0)

// ===========================================================================
// Result rows, device metadata, dump formats
// ===========================================================================

constexpr int RESULT_FORMAT_VERSION = 2;

enum class ResultStatus { Ok, Unsupported, Skipped, Error };

const char *categoryString(Category c);
const char *statusString(ResultStatus s);
Category categoryFromString(const std::string &s);
ResultStatus statusFromString(const std::string &s);
Category categoryFromUnit(const std::string &unit);

struct ResultEntry {
    std::string backend, platform, device, driver;
    std::string category, test, metric, unit;
    ResultStatus status = ResultStatus::Ok;
    float value = 0.0f;
    std::string reason;
    std::string display;
    std::string description;
    std::string metricDescription;

    std::string key() const
    {
        return backend + "/" + platform + "/" + device + "/" + category + "/" + test + "/" + metric;
    }
};

typedef std::vector<ResultEntry> ResultStore;
typedef std::map<std::string, float> BaselineMap;

struct DeviceProp {
    std::string key;
    std::string value;
};

struct DeviceInfo {
    std::string backend, platform, device, driver;
    std::vector<DeviceProp> props;
    std::string key() const { return backend + "/" + platform + "/" + device + "/" + driver; }
};

typedef std::vector<DeviceInfo> DeviceInfoStore;

BaselineMap buildBaselineMap(const ResultStore &store);

bool saveJson(const ResultStore &store, const std::string &filename, const DeviceInfoStore &devices = {});
bool saveCsv(const ResultStore &store, const std::string &filename);
bool saveXml(const ResultStore &store, const std::string &filename, const DeviceInfoStore &devices = {});
std::string resultsToJson(const ResultStore &store, const DeviceInfoStore &devices = {});

ResultStore loadJson(const std::string &filename, DeviceInfoStore *devices = nullptr);
ResultStore loadCsv(const std::string &filename);
ResultStore loadXml(const std::string &filename, DeviceInfoStore *devices = nullptr);
ResultStore loadResultFile(const std::string &filename, DeviceInfoStore *devices = nullptr);

// ===========================================================================
// Logger: scoped emission -> LogEvent stream + accumulated rows
// ===========================================================================

using LogProp = DeviceProp;

struct LogEvent {
    enum class Kind { BackendBegin, DeviceBegin, TestBegin, Metric, TestSkippedAll, TestEnd, DeviceEnd,
                      BackendEnd, Note };
    Kind kind = Kind::Note;
    std::string backend, platform, device, driver;
    std::string testTag, testDisplay, unit;
    Category category = Category::Unknown;
    std::string testDescription;
    std::vector<LogProp> props;          // DeviceBegin
    int platformIndex = -1;
    int deviceIndex = -1;
    bool showPlatformLine = false;
    ResultEntry entry;                   // Metric
    bool subMetric = false;
    std::vector<std::string> metricNames;   // TestSkippedAll
    ResultStatus status = ResultStatus::Ok;
    std::string reason;
    std::string message;                 // Note
};

class logger {
public:
    using Prop = LogProp;

    struct DeviceSpec {
        std::string name;
        std::string platform;            // empty -> the backend name
        std::string driver_version;
        std::vector<Prop> props;
        int platform_index = -1;
        int device_index = -1;
    };

    struct TestSpec {
        std::string tag;
        std::string display;
        std::string unit;
        Category category = Category::Unknown;   // derived from the unit when left Unknown
        std::string description;
    };

    struct EmitOptions {
        bool subMetric = false;
        std::string description;
    };

    class BackendScope;
    class DeviceScope;
    class TestScope;

    BackendScope beginBackend(const std::string &name);
    void note(const std::string &msg);

    bool compareEnabled;
    BaselineMap baseline;
    ResultStore results;
    DeviceInfoStore devices;

    explicit logger(std::string compareFileName = "");
    virtual ~logger() = default;

protected:
    virtual void onEvent(const LogEvent &e) = 0;

    std::string curBackend, curPlatform, curDevice, curDriver;
    std::string curTest, curTestDisplay, curTestDescription, curUnit;
    Category curCategory = Category::Unknown;
    int contextDepth = 0;                // 0 none, 1 backend, 2 device, 3 test
    unsigned long long testSeqCounter = 0;
    unsigned long long curTestSeq = 0;

    void closeOpenTest();

private:
    LogEvent makeEvent(LogEvent::Kind kind) const;
    ResultEntry makeEntry(const std::string &metric, ResultStatus status, float value,
                          const std::string &reason, const std::string &metricDescription = "") const;
    friend class BackendScope;
    friend class DeviceScope;
    friend class TestScope;
};

class logger::BackendScope {
public:
    BackendScope(logger *log, const std::string &name);
    ~BackendScope();
    BackendScope(const BackendScope &) = delete;
    BackendScope &operator=(const BackendScope &) = delete;
    BackendScope(BackendScope &&other) noexcept;
    BackendScope &operator=(BackendScope &&) = delete;
    DeviceScope beginDevice(const DeviceSpec &spec);
    void end();

private:
    logger *log;
    bool closed = false;
};

class logger::DeviceScope {
public:
    DeviceScope(logger *log, const DeviceSpec &spec);
    ~DeviceScope();
    DeviceScope(const DeviceScope &) = delete;
    DeviceScope &operator=(const DeviceScope &) = delete;
    DeviceScope(DeviceScope &&other) noexcept;
    DeviceScope &operator=(DeviceScope &&) = delete;
    TestScope beginTest(const TestSpec &spec);
    void end();

private:
    logger *log;
    bool closed = false;
};

class logger::TestScope {
public:
    TestScope(logger *log, const TestSpec &spec);
    ~TestScope();
    TestScope(const TestScope &) = delete;
    TestScope &operator=(const TestScope &) = delete;
    TestScope(TestScope &&other) noexcept;
    TestScope &operator=(TestScope &&) = delete;
    void emit(std::string metric, float value, EmitOptions opts = {});
    void emit(std::string metric, float value, const char *description);
    void skip(std::string metric, ResultStatus status, std::string reason, std::string description = "");
    void skipAll(std::initializer_list<std::string> metrics, ResultStatus status, std::string reason);
    void end();

private:
    logger *log;
    bool closed = false;
    unsigned long long seq = 0;
};

// Indented text rendering of the event stream (the CLI's output channel).
class LoggerText : public logger {
public:
    explicit LoggerText(std::ostream &out = std::cout, std::string compareFileName = "", bool describe = false)
        : logger(std::move(compareFileName)), out(out), describe(describe)
    {
    }

protected:
    void onEvent(const LogEvent &e) override;
    std::ostream &out;
    bool describe = false;

private:
    struct Row {
        std::string metric;
        float value;
        ResultStatus status;
        std::string reason;
        bool sub;
        std::string key;
        std::string info;
    };
    std::vector<Row> rows;
    int depth = 0;
    int propDepth = 0;
    int metricDepth = 0;
    void flushRows();
    void wrapText(int column, const std::string &text);
};

// ===========================================================================
// Command line
// ===========================================================================

struct CliOptions {
    bool skipOpenCL = false, skipVulkan = false, skipCuda = false, skipRocm = false;
    bool skipMetal = false, skipOneapi = false, skipCpu = false;
    std::vector<unsigned long> platformIndices;
    std::vector<unsigned long> deviceIndices;
    std::vector<int> vkDeviceIndices, cudaDeviceIndices, rocmDeviceIndices, mtlDeviceIndices,
        oneapiDeviceIndices;
    bool forceIters = false;
    unsigned int iters = 0;
    unsigned int warmupCount = 2;
    unsigned int targetTimeUs = DEFAULT_TARGET_TIME_US;
    unsigned int targetTimeUsCpu = DEFAULT_CPU_TARGET_TIME_US;
    std::bitset<static_cast<size_t>(Benchmark::COUNT)> enabledTests;
    std::bitset<static_cast<size_t>(Category::Unknown)> enabledCategories;
    bool useEventTimer = false;
    bool enableXml = false;
    std::string xmlFile;
    bool enableJson = false;
    std::string jsonFile;
    bool enableCsv = false;
    std::string csvFile;
    std::string compareFile;
    bool listDevices = false;
    bool verbose = false;
    bool describe = false;
    // --cpu was given, but this build registers no native CPU backend (backend_table.hpp): the
    // front ends say so and report a non-zero status when nothing else was selected.
    bool namedAbsentBackend = false;

    CliOptions()
    {
        enabledTests.set();
        enabledCategories.set();
    }
};

// Exits on --help / --version / error, like the CLI always did.
int parseCliOptions(int argc, char **argv, CliOptions &out);
// Never exits: false + message on error or on --help / --version.
bool parseCliOptionsNoExit(int argc, char **argv, CliOptions &out, std::string &errorMsg);

// ===========================================================================
// Backend base class
// ===========================================================================

class Peak {
public:
    std::unique_ptr<logger> log;
    unsigned int warmupCount = 2;
    unsigned int specifiedIters = 0;
    unsigned int targetTimeUs = DEFAULT_TARGET_TIME_US;
    bool forceIters = false;
    std::bitset<static_cast<size_t>(Benchmark::COUNT)> enabledTests;
    std::bitset<static_cast<size_t>(Category::Unknown)> enabledCategories;

    Peak()
    {
        enabledTests.set();
        enabledCategories.set();
    }
    virtual ~Peak() = default;

    bool isTestEnabled(Benchmark b) const { return enabledTests.test(static_cast<size_t>(b)); }
    bool isCategoryEnabled(Category c) const
    {
        return c != Category::Unknown && enabledCategories.test(static_cast<size_t>(c));
    }
    bool isAllowed(Benchmark b) const
    {
        return !clpeak::cancelRequested() && isCategoryEnabled(categoryOf(b)) && isTestEnabled(b);
    }
    bool isAllowedAs(Benchmark b, Category c) const
    {
        return !clpeak::cancelRequested() && isCategoryEnabled(c) && isTestEnabled(b);
    }

    virtual void applyOptions(const CliOptions &opts);
    virtual int runAll() = 0;
};

// ===========================================================================
// Device inventory (--list-devices, FFI catalog)
// ===========================================================================

struct InventoryDevice {
    int index = -1;
    std::string name;
    std::string typeStr;
    std::string driverVersion;
    std::string apiVersion;
    unsigned int numComputeUnits = 0;
    unsigned int maxClockMHz = 0;
    std::uint64_t globalMemBytes = 0;
    std::uint64_t maxAllocBytes = 0;
    bool hasFp16 = false;
    bool hasFp64 = false;
};

struct InventoryPlatform {
    int index = -1;
    std::string name;
    std::vector<InventoryDevice> devices;
};

struct BackendInventory {
    std::string backend;
    bool available = false;
    std::vector<InventoryPlatform> platforms;
};

std::string inventoryToJson(const std::vector<BackendInventory> &inv);

#endif // CLPEAK_B200_HOST_API_HPP
