// Host-side helpers shared by the C ABI translation units: the per-thread error message,
// CUDA error capture, and a cached query of the SM count of the current device.
#pragma once
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <string>

#include "../../include/tpb200.h"

namespace tpb {

std::string& last_error_slot();

inline int fail(int code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    last_error_slot() = buf;
    return code;
}

// The reference reports CUDA failures as RuntimeError("CUDA Error: ...")
// (p10/src/backend/cuda/ReductionKernels.cu:21-27); keep the same prefix.
inline int cuda_fail(cudaError_t e, const char* what) {
    return fail(TPB200_ERR_CUDA, "CUDA Error: %s (%s)", cudaGetErrorString(e), what);
}

#define TPB_CUDA_OK(expr)                                            \
    do {                                                             \
        cudaError_t e__ = (expr);                                    \
        if (e__ != cudaSuccess) return ::tpb::cuda_fail(e__, #expr); \
    } while (0)

// Launch check: a bad configuration is reported at once; nothing here waits for the kernel.
#define TPB_LAUNCH_OK(name)                                           \
    do {                                                              \
        cudaError_t e__ = cudaGetLastError();                         \
        if (e__ != cudaSuccess) return ::tpb::cuda_fail(e__, name);   \
    } while (0)

int sm_count();  // SMs of the current device (148 on B200), cached per device
int* device_status_word();  // device address of the per-device status word (nullptr without a device)

// Planner overrides for experiments and tests (TPB200_FORCE_STRATEGY, TPB200_TOPK_SLICES, ...) are
// looked up only when TPB200_EXPERIMENTS was set when the library made its first call; without it
// a call reads no environment variable at all.
bool experiments_on();
inline const char* env_str(const char* name) { return experiments_on() ? getenv(name) : nullptr; }
inline bool env_int(const char* name, int* out) {
    const char* v = env_str(name);
    if (!v || !*v) return false;
    *out = atoi(v);
    return true;
}

inline long long ceil_div(long long a, long long b) { return (a + b - 1) / b; }
inline long long round_up(long long a, long long b) { return ceil_div(a, b) * b; }
inline int pow2_ceil(long long v) {
    int p = 1;
    while (p < v) p <<= 1;
    return p;
}

}  // namespace tpb
