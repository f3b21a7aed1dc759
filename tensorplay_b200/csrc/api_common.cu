// Process-wide pieces of the C ABI: the per-thread error message, the library version and the
// cached SM count that the planners size their grids with.
#include "common.cuh"
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

#ifdef TPB200_CHECKED
// ---- checked build: the range table, the record of the first violation, the sink
__device__ CheckTable g_check_table;
__device__ CheckRecord g_check_record;
__device__ __align__(16) unsigned char g_check_sink[256];

__device__ __noinline__ const void* check_access(const void* p, unsigned bytes, int file, int line) {
    const unsigned long long a = (unsigned long long)p;
    const int n = g_check_table.n;
    for (int i = 0; i < n; ++i)
        if (a >= g_check_table.r[i].lo && a + bytes <= g_check_table.r[i].hi) return p;
    if (atomicCAS(&g_check_record.hit, 0, 1) == 0) {
        g_check_record.file = file;
        g_check_record.line = line;
        g_check_record.bytes = bytes;
        g_check_record.addr = a;
    }
    atomicAdd(&g_check_record.count, 1ull);
    atomicMax(&g_device_status, kErrChecked);
    return g_check_sink;   // the access goes here instead
}

__global__ void check_set_kernel(CheckTable t) { g_check_table = t; }

static long long g_trim_next = 0;

int check_register(cudaStream_t st, const HostRange* r, int n) {
    CheckTable t{};
    if (n > kCheckRanges) return fail(TPB200_ERR_INVALID, "checked build: more than %d ranges in one call", kCheckRanges);
    const long long trim = g_trim_next;
    g_trim_next = 0;
    for (int i = 0; i < n; ++i) {
        if (!r[i].p || r[i].bytes == 0) continue;
        const unsigned long long lo = (unsigned long long)r[i].p;
        unsigned long long hi = lo + r[i].bytes;
        if (trim > 0) hi = hi - lo > (unsigned long long)trim ? hi - (unsigned long long)trim : lo;
        t.r[t.n].lo = lo;
        t.r[t.n].hi = hi;
        ++t.n;
    }
    check_set_kernel<<<1, 1, 0, st>>>(t);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "check_set_kernel");
    return TPB200_OK;
}
#endif

}  // namespace tpb

extern "C" int tpb200_check_report(int64_t* info, int n_info) {
    if (!info || n_info < TPB200_CHECK_INFO_FIELDS) return tpb::fail(TPB200_ERR_INVALID, "info must hold %d fields", TPB200_CHECK_INFO_FIELDS);
    for (int i = 0; i < n_info; ++i) info[i] = 0;
#ifdef TPB200_CHECKED
    tpb::CheckRecord rec{}, zero{};
    TPB_CUDA_OK(cudaMemcpyFromSymbol(&rec, tpb::g_check_record, sizeof(rec)));
    if (rec.hit || rec.count) TPB_CUDA_OK(cudaMemcpyToSymbol(tpb::g_check_record, &zero, sizeof(zero)));
    info[0] = 1;
    info[1] = (int64_t)rec.count;
    info[2] = rec.file;
    info[3] = rec.line;
    info[4] = (int64_t)rec.addr;
    info[5] = rec.bytes;
#endif
    return TPB200_OK;
}

extern "C" int tpb200_check_trim_next(int64_t bytes) {
#ifdef TPB200_CHECKED
    if (bytes < 0) return tpb::fail(TPB200_ERR_INVALID, "bytes must not be negative");
    tpb::g_trim_next = bytes;
    return TPB200_OK;
#else
    (void)bytes;
    return tpb::fail(TPB200_ERR_UNSUPPORTED, "this library was built without -DTPB200_CHECKED");
#endif
}

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
