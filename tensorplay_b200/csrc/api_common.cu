// Process-wide pieces of the C ABI: the per-thread error message, the library version and the
// cached SM count that the planners size their grids with.
#include "host_util.h"

#include <mutex>

namespace tpb {

std::string& last_error_slot() {
    static thread_local std::string msg;
    return msg;
}

bool experiments_on() {
    static const bool on = getenv("TPB200_EXPERIMENTS") != nullptr;   // read once
    return on;
}

int sm_count() {
    static std::mutex mu;
    static int cached[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
        (void)cudaGetLastError();
        return 148;  // B200; only reached without a usable device (e.g. a workspace-size query)
    }
    std::lock_guard<std::mutex> lk(mu);
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) {
            (void)cudaGetLastError();
            n = 148;
        }
        cached[dev] = n;
    }
    return cached[dev];
}

// Set by a kernel whose bounded wait gave up (its outputs are then not written): top-k rendezvous /
// polling, or the peer exchange of the fused sharded reduction.  One word per device, in the
// module's global memory; kernels get its address as a plain pointer.
__device__ int g_device_status = 0;

int* device_status_word() {
    static std::mutex mu;
    static int* cached[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { (void)cudaGetLastError(); return nullptr; }
    std::lock_guard<std::mutex> lk(mu);
    if (!cached[dev]) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_device_status) != cudaSuccess) { (void)cudaGetLastError(); return nullptr; }
        cached[dev] = (int*)p;
    }
    return cached[dev];
}

}  // namespace tpb

extern "C" int tpb200_device_status(int* status_out) {
    if (!status_out) return tpb::fail(TPB200_ERR_INVALID, "status_out is NULL");
    int v = 0, zero = 0;
    TPB_CUDA_OK(cudaMemcpyFromSymbol(&v, tpb::g_device_status, sizeof(int)));
    if (v != 0) TPB_CUDA_OK(cudaMemcpyToSymbol(tpb::g_device_status, &zero, sizeof(int)));
    *status_out = v;
    return TPB200_OK;
}

extern "C" const char* tpb200_last_error(void) { return tpb::last_error_slot().c_str(); }
extern "C" int tpb200_version(void) { return TPB200_VERSION; }
