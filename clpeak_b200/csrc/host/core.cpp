// Small shared pieces of the host contract: calibration, cancel / verbose
// flags, enum <-> string tables, option hand-over to a backend, inventory JSON.
#include <atomic>
#include <cstring>
#include <locale>
#include <sstream>

#include "clpeak_api.hpp"

namespace clpeak {
namespace {
std::atomic<bool> g_cancel{false};
std::atomic<bool> g_verbose{false};
} // namespace
bool verboseEnabled() { return g_verbose.load(std::memory_order_relaxed); }
void setVerbose(bool on) { g_verbose.store(on, std::memory_order_relaxed); }
void requestCancel() { g_cancel.store(true, std::memory_order_relaxed); }
bool cancelRequested() { return g_cancel.load(std::memory_order_relaxed); }
void resetCancel() { g_cancel.store(false, std::memory_order_relaxed); }
} // namespace clpeak

// Same contract as the reference's pickIters (src/common/common.cpp:35-45).
unsigned int pickIters(double per_iter_us, unsigned int target_us, unsigned int forced, unsigned int max_iters)
{
    if (forced != 0)
        return forced;
    const double budget = target_us ? (double)target_us : 5.0e6;
    const double one = per_iter_us < 1.0 ? 1.0 : per_iter_us;
    double n = budget / one;
    n = std::max(1.0, std::min(n, (double)max_iters));
    return (unsigned int)n;
}

benchmark_config_t benchmark_config_t::forDevice(DeviceType type)
{
    const bool cpu = (type == DeviceType::Cpu);
    benchmark_config_t c;
    c.globalBWMaxSize = cpu ? (1ull << 27) : (1ull << 29);
    c.transferBWMaxSize = c.globalBWMaxSize;
    c.computeWgsPerCU = cpu ? 512 : 2048;
    c.computeDPWgsPerCU = cpu ? 256 : 512;
    c.targetTimeUs = DEFAULT_TARGET_TIME_US;
    c.kernelLatencyIters = 2000;
    return c;
}

// xorshift32 bit patterns forced into the finite float range
// (src/common/common.cpp:76-95).  Kept for host-side callers of the contract;
// the B200 backend fills its buffers on the device instead.
void populate(float *ptr, uint64_t N)
{
    uint32_t s = 0xDEADBEEFu;
    for (uint64_t i = 0; i < N; ++i) {
        s ^= s << 13;
        s ^= s >> 17;
        s ^= s << 5;
        const uint32_t bits = (s & 0x7F7FFFFFu) | 0x00800000u;
        std::memcpy(ptr + i, &bits, sizeof(bits));
    }
}

std::string jsonEscape(const std::string &in)
{
    std::string out;
    out.reserve(in.size() + 8);
    for (unsigned char ch : in) {
        switch (ch) {
        case '"': out += "\\\""; break;
        case '\\': out += "\\\\"; break;
        case '\n': out += "\\n"; break;
        case '\r': out += "\\r"; break;
        case '\t': out += "\\t"; break;
        default:
            if (ch < 0x20) {
                char buf[8];
                std::snprintf(buf, sizeof(buf), "\\u%04x", (unsigned)ch);
                out += buf;
            } else {
                out += (char)ch;
            }
        }
    }
    return out;
}

namespace {
struct CatName { Category c; const char *s; };
const CatName kCats[] = {
    {Category::FpCompute, "fp_compute"}, {Category::IntCompute, "int_compute"}, {Category::Crypto, "crypto"},
    {Category::String, "string"},        {Category::Bandwidth, "bandwidth"},    {Category::Latency, "latency"},
};
struct StatName { ResultStatus st; const char *s; };
const StatName kStats[] = {
    {ResultStatus::Ok, "ok"}, {ResultStatus::Unsupported, "unsupported"}, {ResultStatus::Skipped, "skipped"},
    {ResultStatus::Error, "error"},
};
} // namespace

const char *categoryString(Category c)
{
    for (const auto &e : kCats)
        if (e.c == c)
            return e.s;
    return "";
}

Category categoryFromString(const std::string &s)
{
    for (const auto &e : kCats)
        if (s == e.s)
            return e.c;
    return Category::Unknown;
}

const char *statusString(ResultStatus st)
{
    for (const auto &e : kStats)
        if (e.st == st)
            return e.s;
    return "ok";
}

ResultStatus statusFromString(const std::string &s)
{
    for (const auto &e : kStats)
        if (s == e.s)
            return e.st;
    return ResultStatus::Ok;
}

Category categoryFromUnit(const std::string &u)
{
    if (u == "gflops" || u == "tflops") return Category::FpCompute;
    if (u == "gops" || u == "tops") return Category::IntCompute;
    if (u == "gbps") return Category::Bandwidth;
    if (u == "us") return Category::Latency;
    return Category::Unknown;
}

BaselineMap buildBaselineMap(const ResultStore &store)
{
    BaselineMap m;
    for (const auto &row : store)
        if (row.status == ResultStatus::Ok)
            m[row.key()] = row.value;
    return m;
}

void Peak::applyOptions(const CliOptions &o)
{
    forceIters = o.forceIters;
    specifiedIters = o.iters;
    warmupCount = o.warmupCount;
    targetTimeUs = o.targetTimeUs;
    enabledTests = o.enabledTests;
    enabledCategories = o.enabledCategories;
}

std::string inventoryToJson(const std::vector<BackendInventory> &inv)
{
    std::ostringstream os;
    os.imbue(std::locale::classic());
    os << "{\"backends\":[";
    bool firstB = true;
    for (const auto &b : inv) {
        os << (firstB ? "" : ",") << "{\"name\":\"" << jsonEscape(b.backend) << "\",\"available\":"
           << (b.available ? "true" : "false") << ",\"platforms\":[";
        firstB = false;
        bool firstP = true;
        for (const auto &p : b.platforms) {
            os << (firstP ? "" : ",") << "{\"index\":" << p.index << ",\"name\":\"" << jsonEscape(p.name)
               << "\",\"devices\":[";
            firstP = false;
            bool firstD = true;
            for (const auto &d : p.devices) {
                os << (firstD ? "" : ",") << "{\"index\":" << d.index << ",\"name\":\"" << jsonEscape(d.name)
                   << "\",\"type\":\"" << jsonEscape(d.typeStr) << "\"";
                firstD = false;
                if (!d.driverVersion.empty()) os << ",\"driver\":\"" << jsonEscape(d.driverVersion) << "\"";
                if (!d.apiVersion.empty()) os << ",\"api\":\"" << jsonEscape(d.apiVersion) << "\"";
                if (d.numComputeUnits) os << ",\"computeUnits\":" << d.numComputeUnits;
                if (d.maxClockMHz) os << ",\"clockMHz\":" << d.maxClockMHz;
                if (d.globalMemBytes) os << ",\"globalMemBytes\":" << d.globalMemBytes;
                if (d.maxAllocBytes) os << ",\"maxAllocBytes\":" << d.maxAllocBytes;
                if (d.hasFp16) os << ",\"fp16\":true";
                if (d.hasFp64) os << ",\"fp64\":true";
                os << "}";
            }
            os << "]}";
        }
        os << "]}";
    }
    os << "]}";
    return os.str();
}
