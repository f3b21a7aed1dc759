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

// Programmatic dependent launch of the sampled-threshold top-k kernel: off unless TPB200_PDL=1 (with
// TPB200_EXPERIMENTS set).  Measured on one B200, kernels back to back in one CUDA graph: it bought
// 0.2 us of 33 us on [256,151936] k = 50 and 2 us of 162 us on a 2^28-element sum, nothing on the
// [4096,4096] row reductions, and the two griddepcontrol instructions at the top of a kernel cost
// every CTA about 2 us on kernels of many short CTAs ([64,4096,512] summed over dims (0,2): 76.5 us
// without them, 94.8 us with them, whether or not the launch carried the attribute).  The reductions
// therefore launch the ordinary way and execute no such instruction.
inline bool dependent_launch_on() {
    int v = 0;
    env_int("TPB200_PDL", &v);
    return v != 0;
}

// One launch through cudaLaunchKernelEx.  `cluster` > 1 makes clusters of that many CTAs along x.
// `dependent` lets the kernel start before the previous kernel of the stream has finished; such a
// kernel must wait (griddepcontrol.wait) before it touches memory.
template <class... KArgs, class... Args>
inline cudaError_t launch_ex(void (*kernel)(KArgs...), dim3 grid, int threads, size_t smem, cudaStream_t st,
                             int cluster, bool dependent, Args... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = dim3((unsigned)threads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    unsigned na = 0;
    if (cluster > 1) {
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = (unsigned)cluster;
        attr[na].val.clusterDim.y = 1;
        attr[na].val.clusterDim.z = 1;
        ++na;
    }
    if (dependent) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

#define TPB_LAUNCH(name, kernel, grid, threads, smem, st, ...)                                                    \
    do {                                                                                                          \
        cudaError_t e__ = ::tpb::launch_ex(kernel, grid, threads, smem, st, 1, false, __VA_ARGS__);                 \
        if (e__ != cudaSuccess) return ::tpb::cuda_fail(e__, name);                                               \
    } while (0)

// Checked build (-DTPB200_CHECKED): every entry point registers the address ranges its kernels may
// touch before it launches them -- a one-thread kernel on the same stream writes the table, so the
// registration is ordered with the launches and can be captured in a graph.  One table per device:
// calls on different streams of one device must not overlap in a checked build.
struct HostRange { const void* p; size_t bytes; };
inline HostRange view_range(const void* base, int ndim, const int64_t* sizes, const int64_t* strides, size_t elem) {
    long long lo = 0, hi = 0;
    for (int i = 0; i < ndim; ++i) {
        if (sizes[i] == 0) return HostRange{base, 0};
        const long long span = (long long)(sizes[i] - 1) * (long long)strides[i];
        if (span < 0) lo += span; else hi += span;
    }
    return HostRange{(const char*)base + lo * (long long)elem, (size_t)(hi - lo + 1) * elem};
}
#ifdef TPB200_CHECKED
int check_register(cudaStream_t st, const HostRange* r, int n);
#define TPB_CHECK_RANGES(st, ...)                                                            \
    do {                                                                                     \
        const ::tpb::HostRange r__[] = {__VA_ARGS__};                                        \
        const int rc__ = ::tpb::check_register((st), r__, (int)(sizeof(r__) / sizeof(r__[0]))); \
        if (rc__ != TPB200_OK) return rc__;                                                  \
    } while (0)
#else
#define TPB_CHECK_RANGES(st, ...) do { } while (0)
#endif

inline long long ceil_div(long long a, long long b) { return (a + b - 1) / b; }
inline long long round_up(long long a, long long b) { return ceil_div(a, b) * b; }
inline int pow2_ceil(long long v) {
    int p = 1;
    while (p < v) p <<= 1;
    return p;
}

}  // namespace tpb
