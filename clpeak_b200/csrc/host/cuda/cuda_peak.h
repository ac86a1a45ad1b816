// The "CUDA" backend slot of clpeak, filled by the sm_100a (B200) backend.
//
// Same registration surface as the reference's CudaPeak
// (include/cuda/cuda_peak.h:161-210): a default-constructible Peak subclass with
// applyOptions / runAll and the static enumerate / printInventory pair, so the
// two backend tables (src/cli/main.cpp:54-65, src/ffi/clpeak_ffi.cpp:65-70) take
// it unchanged.  Everything below that surface is different: kernels are reached
// through the C ABI of clpeak_b200_kernels.h instead of embedded fatbins and the
// driver API, every selected GPU runs the test list concurrently on its own host
// thread and stream, and every reading is checked against a host reference of the
// same math before it is reported.
#ifndef CLPEAK_B200_CUDA_PEAK_H
#define CLPEAK_B200_CUDA_PEAK_H

#include <ostream>
#include <string>
#include <vector>

#include <common/inventory.h>
#include <common/peak.h>

struct cuda_device_info_t {
    std::string deviceName;
    std::string driverVersion;     // "13.0"
    std::string runtimeVersion;    // "12.9"
    std::string archName;          // "sm_100"
    int numSMs = 0;
    uint64_t totalGlobalMem = 0;
    int ccMajor = 0, ccMinor = 0;
    int index = -1;
};

// One row a worker produced for a test; turned into emit()/skip() on the
// launching thread.
struct B200Reading {
    std::string metric;
    ResultStatus status = ResultStatus::Ok;
    float value = 0.0f;
    std::string reason;
    std::string info;          // per-reading note (roofline fraction, variant, check outcome)
    double work = 0.0;         // units of work per launch and seconds per launch,
    double seconds = 0.0;      // kept so box aggregates can be formed as sum(work) / max(time)
};

struct B200TestResult {
    logger::TestSpec spec;
    std::vector<B200Reading> readings;
};

class CudaPeak : public Peak {
public:
    CudaPeak();
    ~CudaPeak() override;

    void applyOptions(const CliOptions &opts) override;
    int runAll() override;

    static BackendInventory enumerate();
    static void printInventory(const BackendInventory &b, std::ostream &os);

    // Start-barrier timeout for the per-test rendezvous of the device threads.
    unsigned int barrierTimeoutMs = 120000;

private:
    std::vector<int> deviceIndices;        // --cuda-device (empty = all)
    friend struct B200Harness;
};

#endif // CLPEAK_B200_CUDA_PEAK_H
