// Shared by every .cu in the shim: status plumbing and launch helpers.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/clpeak_b200_kernels.h"

namespace clpk {

// Record a detail string for clpk_last_error() (thread-local).
void set_error(const char *fmt, ...);

// Maps a CUDA error to CLPK_ERR_CUDA / CLPK_ERR_NO_DEVICE and records the detail.
int cuda_fail(cudaError_t e, const char *what);

// The current device must be compute capability 10.x; anything else is refused
// (there is no fallback path).
int require_sm100();

int num_sms();          // of the current device (cached per device)
int smem_optin_bytes(); // of the current device

// Value of a CLPK_TUNE_* knob, or -1 when neither the environment (read once) nor
// clpk_set_tuning has set it.
int tuning(int knob);

// fp32 (CUDA cores) and fp64 (DMMA) GEMMs, simt_gemm.cu; dtype is CLPK_DT_F32 or CLPK_DT_F64.
int launch_simt_gemm(int dtype, const void *a, const void *b, void *c, uint32_t m, uint32_t n, uint32_t k, float alpha,
                     cudaStream_t s);

inline cudaStream_t as_stream(void *s) { return reinterpret_cast<cudaStream_t>(s); }

} // namespace clpk

#define CLPK_CUDA(call)                                          \
    do {                                                         \
        cudaError_t e__ = (call);                                \
        if (e__ != cudaSuccess)                                  \
            return ::clpk::cuda_fail(e__, #call);                \
    } while (0)

#define CLPK_REQUIRE(cond, ...)                                  \
    do {                                                         \
        if (!(cond)) {                                           \
            ::clpk::set_error(__VA_ARGS__);                      \
            return CLPK_ERR_BAD_ARG;                             \
        }                                                        \
    } while (0)

#define CLPK_LAUNCH_CHECK(name)                                  \
    do {                                                         \
        cudaError_t e__ = cudaGetLastError();                    \
        if (e__ != cudaSuccess)                                  \
            return ::clpk::cuda_fail(e__, "launch " name);       \
    } while (0)
