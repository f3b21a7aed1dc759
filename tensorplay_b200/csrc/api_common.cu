// Process-wide pieces of the C ABI: the per-thread error message, the library version and the
// cached SM count that the planners size their grids with.
#include "host_util.h"

#include <mutex>

namespace tpb {

std::string& last_error_slot() {
    static thread_local std::string msg;
    return msg;
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

}  // namespace tpb

extern "C" const char* tpb200_last_error(void) { return tpb::last_error_slot().c_str(); }
extern "C" int tpb200_version(void) { return TPB200_VERSION; }
