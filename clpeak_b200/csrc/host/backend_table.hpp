// The backend registry shared by the CLI and the FFI entry points: name,
// inventory, factory and the CliOptions skip switch, in registration order
// (the reference keeps two mirrored copies of this table, src/cli/main.cpp:39-139
// and src/ffi/clpeak_ffi.cpp:54-108).  This build carries the CUDA slot only.
#pragma once

#include <functional>
#include <memory>
#include <vector>

#include <cuda/cuda_peak.h>
#include <common/options.h>

struct ClpeakBackend {
    const char *name;
    std::function<BackendInventory()> enumerate;
    std::function<void(const BackendInventory &, std::ostream &)> printInventory;
    std::function<std::unique_ptr<Peak>()> create;
    bool CliOptions::*skip;
};

inline const std::vector<ClpeakBackend> &clpeakBackends()
{
    static const std::vector<ClpeakBackend> table = {
        {"CUDA", [] { return CudaPeak::enumerate(); },
         [](const BackendInventory &b, std::ostream &os) { CudaPeak::printInventory(b, os); },
         [] { return std::unique_ptr<Peak>(new CudaPeak()); }, &CliOptions::skipCuda},
    };
    return table;
}
