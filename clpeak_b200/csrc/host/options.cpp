// Command-line grammar of clpeak, for the flag set a CUDA + CPU build of the
// reference accepts (src/common/options.cpp): --<backend> / --no-<backend>,
// --cuda-device <list>, -i / -w / --max-time / --max-time-cpu, the output
// files, four category flags and the per-test flags with their --no- forms.
//
// Selection semantics kept from the reference (options.cpp:391-434): the first
// positive --<test> flag switches the test set from "everything" to "only what
// is named"; --no-<test> always subtracts; categories work the same way; any
// positive --<backend> flag means "only the named backends".  Unknown flags are
// errors.  Flags of backends this build does not carry (--vulkan, --rocm ...)
// are unknown here exactly as they are in a reference binary built without them.
#include <cerrno>
#include <cstdlib>
#include <cstring>
#include <limits>
#include <sstream>

#include "clpeak_api.hpp"

namespace {

const char *kHelp = R"( clpeak [OPTIONS]   (B200 / sm_100a CUDA backend)

 GLOBAL OPTIONS:
  -h, --help                  display help message
  -v, --version               display version
  -i, --iters num             force a fixed iter count (overrides --max-time calibration)
  -w, --warmup num            number of warm-up kernel runs before timing (default: 2)
  --max-time ms               per-test time budget for the timed phase (default: 500 ms)
  --max-time-cpu ms           per-test time budget for the CPU backend (accepted, unused: no CPU backend here)
  --verbose                   print backend debug logs
  --describe                  explain what each test and each reading measures
  --list-devices              list available devices for every backend and exit
  --xml-file file             save results to an XML file
  --json-file file            save results to a JSON file
  --csv-file file             save results to a CSV file
  --compare file              compare results against a baseline (JSON / CSV / XML)

 BACKEND SELECTION (default: run every available backend):
  --cuda / --no-cuda          run only / skip the CUDA backend
  --cpu  / --no-cpu           accepted for scripts written for a full clpeak build; this build carries
                              the CUDA backend only, so --cpu alone runs nothing and exits non-zero
  --cuda-device list          comma-separated CUDA device indices (default: all, run concurrently)

 CATEGORY SELECTION (--<cat> runs only the named categories, --no-<cat> removes one):
  --fp-compute  --int-compute  --crypto  --string  --bandwidth  --latency

 TEST SELECTION (--<test> runs only the named tests, --no-<test> removes one):
  --single-precision-compute  --half-precision-compute  --double-precision-compute
  --mixed-precision-compute   --bfloat16-compute        --integer-compute
  --int8-dot-product-compute  --wmma                    --cublas
  --global-memory-bandwidth   --local-memory-bandwidth  --image-memory-bandwidth
  --transfer-bandwidth        --kernel-launch-latency   --memory-latency
)";

struct NamedTest { const char *flag; Benchmark test; };
const NamedTest kTests[] = {
    {"single-precision-compute", Benchmark::ComputeSP},
    {"half-precision-compute", Benchmark::ComputeHP},
    {"double-precision-compute", Benchmark::ComputeDP},
    {"mixed-precision-compute", Benchmark::ComputeMP},
    {"bfloat16-compute", Benchmark::ComputeBF16},
    {"integer-compute", Benchmark::ComputeInt},
    {"int8-dot-product-compute", Benchmark::ComputeInt8DP},
    {"int16-dot-product-compute", Benchmark::ComputeInt16DP},
    {"fp8-dot-product-compute", Benchmark::ComputeFP8DP},
    {"divide-sqrt-compute", Benchmark::ComputeDivSqrt},
    {"integer-divide-compute", Benchmark::ComputeIntDiv},
    {"wmma", Benchmark::Wmma},
    {"cublas", Benchmark::Cublas},
    {"amx", Benchmark::Amx},
    {"accelerate", Benchmark::AppleBlas},
    {"aes", Benchmark::CryptoAes},
    {"sha256", Benchmark::CryptoSha256},
    {"sha512", Benchmark::CryptoSha512},
    {"crc32c", Benchmark::CryptoCrc32c},
    {"string-scan", Benchmark::StringScan},
    {"utf8-validate", Benchmark::Utf8Validate},
    {"cache-bandwidth", Benchmark::CacheBandwidth},
    {"memory-latency", Benchmark::MemoryLatency},
    {"atomics", Benchmark::Atomics},
    {"branch-penalty", Benchmark::BranchPenalty},
    {"store-forward", Benchmark::StoreForward},
    {"smt-scaling", Benchmark::SmtScaling},
    {"global-memory-bandwidth", Benchmark::GlobalBW},
    {"local-memory-bandwidth", Benchmark::LocalBW},
    {"image-memory-bandwidth", Benchmark::ImageBW},
    {"transfer-bandwidth", Benchmark::TransferBW},
    {"kernel-launch-latency", Benchmark::KernelLatency},
};

struct NamedCategory { const char *flag; Category cat; };
const NamedCategory kCategories[] = {
    {"fp-compute", Category::FpCompute}, {"int-compute", Category::IntCompute}, {"crypto", Category::Crypto},
    {"string", Category::String},        {"bandwidth", Category::Bandwidth},    {"latency", Category::Latency},
};

enum class Outcome { Ok, Help, Version, Error };

bool toULong(const char *text, unsigned long &v)
{
    char *end = nullptr;
    errno = 0;
    v = std::strtoul(text, &end, 0);
    return errno != ERANGE && end != text && *end == '\0';
}

bool toUInt(const char *text, unsigned int &v, bool zeroOk)
{
    unsigned long p;
    if (!toULong(text, p) || p > std::numeric_limits<unsigned int>::max() || (!zeroOk && p == 0))
        return false;
    v = (unsigned int)p;
    return true;
}

bool toIndexList(const char *text, std::vector<int> &out)
{
    std::vector<int> parsed;
    std::stringstream ss(text);
    std::string tok;
    while (std::getline(ss, tok, ',')) {
        unsigned long v;
        if (tok.empty() || !toULong(tok.c_str(), v) || v > (unsigned long)std::numeric_limits<int>::max())
            return false;
        parsed.push_back((int)v);
    }
    if (parsed.empty())
        return false;
    out.swap(parsed);
    return true;
}

// "--name" -> (name, false); "--no-name" -> (name, true); anything else -> empty name.
std::string flagBody(const char *arg, bool &negated)
{
    negated = false;
    if (std::strncmp(arg, "--", 2) != 0)
        return {};
    const char *body = arg + 2;
    if (std::strncmp(body, "no-", 3) == 0) {
        negated = true;
        body += 3;
    }
    return body;
}

Outcome parse(int argc, char **argv, CliOptions &o, std::string &err)
{
    bool onlyNamedBackends = false, wantCuda = false, wantCpu = false;
    bool testsNarrowed = false, categoriesNarrowed = false;

    auto value = [&](int &i) -> const char * { return (i + 1 < argc) ? argv[++i] : nullptr; };
    auto missing = [&](const char *flag) {
        err = std::string("clpeak: missing argument for ") + flag + "\n";
        return Outcome::Error;
    };
    auto invalid = [&](const char *flag, const char *v) {
        err = std::string("clpeak: invalid value for ") + flag + ": " + v + "\n";
        return Outcome::Error;
    };

    for (int i = 1; i < argc; ++i) {
        const char *a = argv[i];
        const std::string s = a;
        if (s == "-h" || s == "--help")
            return Outcome::Help;
        if (s == "-v" || s == "--version")
            return Outcome::Version;
        if (s == "--verbose") { o.verbose = true; continue; }
        if (s == "--describe") { o.describe = true; continue; }
        if (s == "--list-devices") { o.listDevices = true; continue; }
        if (s == "--cuda") { wantCuda = onlyNamedBackends = true; continue; }
        if (s == "--no-cuda") { o.skipCuda = true; continue; }
        if (s == "--cpu") { wantCpu = onlyNamedBackends = o.namedAbsentBackend = true; continue; }
        if (s == "--no-cpu") { o.skipCpu = true; continue; }

        if (s == "-i" || s == "--iters") {
            const char *v = value(i);
            if (!v) return missing(a);
            unsigned int n;
            if (!toUInt(v, n, false)) return invalid(a, v);
            o.forceIters = true;
            o.iters = n;
            continue;
        }
        if (s == "-w" || s == "--warmup") {
            const char *v = value(i);
            if (!v) return missing(a);
            unsigned int n;
            if (!toUInt(v, n, true)) return invalid(a, v);
            o.warmupCount = n;
            continue;
        }
        if (s == "--max-time" || s == "--max-time-cpu") {
            const char *v = value(i);
            if (!v) return missing(a);
            unsigned int ms;
            if (!toUInt(v, ms, false) || ms > std::numeric_limits<unsigned int>::max() / 1000u)
                return invalid(a, v);
            (s == "--max-time" ? o.targetTimeUs : o.targetTimeUsCpu) = ms * 1000u;
            continue;
        }
        if (s == "--cuda-device") {
            const char *v = value(i);
            if (!v) return missing(a);
            if (!toIndexList(v, o.cudaDeviceIndices)) {
                err = std::string("clpeak: invalid CUDA device index list: ") + v + "\n";
                return Outcome::Error;
            }
            continue;
        }
        if (s == "--xml-file" || s == "--json-file" || s == "--csv-file" || s == "--compare") {
            const char *v = value(i);
            if (!v) return missing(a);
            if (s == "--xml-file") { o.xmlFile = v; o.enableXml = true; }
            else if (s == "--json-file") { o.jsonFile = v; o.enableJson = true; }
            else if (s == "--csv-file") { o.csvFile = v; o.enableCsv = true; }
            else o.compareFile = v;
            continue;
        }

        bool negated = false;
        const std::string body = flagBody(a, negated);
        bool matched = false;
        if (!body.empty()) {
            for (const auto &c : kCategories) {
                if (body != c.flag)
                    continue;
                if (!negated && !categoriesNarrowed) {
                    o.enabledCategories.reset();
                    categoriesNarrowed = true;
                }
                o.enabledCategories.set((size_t)c.cat, !negated);
                matched = true;
                break;
            }
            for (size_t t = 0; !matched && t < sizeof(kTests) / sizeof(kTests[0]); ++t) {
                if (body != kTests[t].flag)
                    continue;
                if (!negated && !testsNarrowed) {
                    o.enabledTests.reset();
                    testsNarrowed = true;
                }
                o.enabledTests.set((size_t)kTests[t].test, !negated);
                matched = true;
            }
        }
        if (!matched) {
            err = std::string("clpeak: unknown option '") + a + "'\n";
            return Outcome::Error;
        }
    }

    if (onlyNamedBackends) {
        o.skipOpenCL = o.skipVulkan = o.skipRocm = o.skipMetal = o.skipOneapi = true;
        if (!wantCuda) o.skipCuda = true;
        if (!wantCpu) o.skipCpu = true;
    }
    return Outcome::Ok;
}

} // namespace

int parseCliOptions(int argc, char **argv, CliOptions &out)
{
    std::string err;
    switch (parse(argc, argv, out, err)) {
    case Outcome::Ok:
        return 0;
    case Outcome::Help:
        std::cout << kHelp << "\n";
        std::cout.flush();
        std::exit(0);
    case Outcome::Version:
        std::cout << "clpeak version: " << CLPEAK_VERSION_STR << "\n";
        std::exit(0);
    case Outcome::Error:
        std::cerr << err;
        std::cout << kHelp << "\n";
        std::cout.flush();
        std::exit(-1);
    }
    return 0;
}

bool parseCliOptionsNoExit(int argc, char **argv, CliOptions &out, std::string &errorMsg)
{
    switch (parse(argc, argv, out, errorMsg)) {
    case Outcome::Ok:
        return true;
    case Outcome::Help:
        errorMsg = "clpeak: --help is not available when embedded\n";
        return false;
    case Outcome::Version:
        errorMsg = "clpeak: --version is not available when embedded\n";
        return false;
    case Outcome::Error:
        return false;
    }
    return false;
}
