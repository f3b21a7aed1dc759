// Single-process multi-GPU host of the sharded paths, in the C ABI: tpb200_comm_create / _destroy,
// tpb200_reduce_sharded, tpb200_topk_sharded.  A C++ TensorPlay host needs nothing else -- no
// Python, no PyTorch -- to run a whole-tensor reduction or a global top-k over a flat tensor whose
// partitions live on several GPUs of one box.  The reference has no multi-GPU support at all (its
// allocator pins device 0: p10/src/backend/cuda/CUDAAllocator.cpp:87-88), so the contract is "the
// answer of the one-GPU kernel on the un-sharded tensor, identical on every GPU".
//
// A comm owns, per GPU: a stream, an exchange buffer for the fused reduction (peer-mapped), scratch
// for the slice kernels and the local top-k, a gather buffer for records and top-k candidates, and
// events.  Everything is allocated in tpb200_comm_create; the calls themselves only enqueue work.
//
//   distinct GPUs with peer access   whole-tensor reductions run tpb200_reduce_fused_exchange on every
//                                    GPU: the 40-byte records cross NVLink by plain peer stores inside
//                                    the kernels, no copy engine and no library collective
//   otherwise (e.g. the same GPU     every partition is reduced to its record, the records are copied
//   listed several times: tests)     into every GPU's gather buffer, and tpb200_reduce_combine merges
//                                    them in rank order.  Kernels of different ranks never wait on
//                                    one another in this mode, so it is safe on a single GPU.
//   global top-k                     local top-k per GPU, candidate lists copied to every GPU's gather
//                                    buffer (cudaMemcpyPeerAsync, ordered by events), tpb200_topk_merge
//                                    with the partition offsets applied in the kernel.
#include "host_util.h"

// A checked build keeps one range table per device: where several logical GPUs of a comm share a device,
// their calls must not overlap, so each one is waited for.  (The fused mode needs distinct devices.)
#ifdef TPB200_CHECKED
#define TPB_CHECKED_SERIALIZE(st) TPB_CUDA_OK(cudaStreamSynchronize(st))
#else
#define TPB_CHECKED_SERIALIZE(st) do { } while (0)
#endif

#include <algorithm>
#include <new>
#include <vector>

namespace tpb {

constexpr int kCommMaxGpus = 16;
constexpr size_t kCommScratchBytes = 8u << 20;     // slice records and top-k slice survivors
constexpr int kCommMaxK = 2048;

struct CommGpu {
    int device = 0;
    cudaStream_t stream = nullptr;
    void* exchange = nullptr;        // tpb200_exchange_buffer_bytes()
    void* scratch = nullptr;         // kCommScratchBytes
    unsigned char* records = nullptr;   // n * TPB200_PARTIAL_BYTES
    float* cand_val = nullptr;       // n * kCommMaxK
    int64_t* cand_idx = nullptr;     // n * kCommMaxK
    int64_t* offsets = nullptr;      // n
    float* out_val = nullptr;        // kCommMaxK (results when the caller passes no buffer)
    int64_t* out_idx = nullptr;      // kCommMaxK
    cudaEvent_t ready = nullptr;     // this GPU's local result is complete
    cudaEvent_t gathered = nullptr;  // everything copied into this GPU's gather buffer has arrived
};

}  // namespace tpb

struct tpb200_comm {
    int n = 0;
    bool fused = false;
    std::vector<tpb::CommGpu> g;
};

using namespace tpb;

namespace {

struct DeviceGuard {
    int prev = 0;
    DeviceGuard() { cudaGetDevice(&prev); }
    ~DeviceGuard() { cudaSetDevice(prev); }
};

int family_of_op(int op) {
    switch (op) {
        case TPB200_OP_SUM: case TPB200_OP_MEAN: return TPB200_OP_SUM;
        case TPB200_OP_VAR: case TPB200_OP_STD: return TPB200_OP_VAR;
        case TPB200_OP_MAX: case TPB200_OP_ARGMAX: case TPB200_OP_MAX_ARGMAX: return TPB200_OP_MAX_ARGMAX;
        case TPB200_OP_MIN: case TPB200_OP_ARGMIN: case TPB200_OP_MIN_ARGMIN: return TPB200_OP_MIN_ARGMIN;
        default: return -1;
    }
}

void free_gpu(CommGpu& c) {
    cudaSetDevice(c.device);
    if (c.stream) cudaStreamSynchronize(c.stream);
    cudaFree(c.exchange); cudaFree(c.scratch); cudaFree(c.records); cudaFree(c.cand_val);
    cudaFree(c.cand_idx); cudaFree(c.offsets); cudaFree(c.out_val); cudaFree(c.out_idx);
    if (c.ready) cudaEventDestroy(c.ready);
    if (c.gathered) cudaEventDestroy(c.gathered);
    if (c.stream) cudaStreamDestroy(c.stream);
    c = CommGpu{};
}

}  // namespace

extern "C" int tpb200_comm_create(int n_gpus, const int* devices, tpb200_comm** out) {
    if (!out) return fail(TPB200_ERR_INVALID, "out is NULL");
    *out = nullptr;
    if (n_gpus < 1 || n_gpus > kCommMaxGpus) return fail(TPB200_ERR_UNSUPPORTED, "1..%d GPUs are supported, %d given", kCommMaxGpus, n_gpus);
    if (!devices) return fail(TPB200_ERR_INVALID, "devices is NULL");
    int count = 0;
    TPB_CUDA_OK(cudaGetDeviceCount(&count));
    bool distinct = true;
    for (int i = 0; i < n_gpus; ++i) {
        if (devices[i] < 0 || devices[i] >= count) return fail(TPB200_ERR_INVALID, "device %d does not exist (%d devices)", devices[i], count);
        for (int j = 0; j < i; ++j) distinct = distinct && devices[j] != devices[i];
    }
    DeviceGuard guard;
    tpb200_comm* c = new (std::nothrow) tpb200_comm;
    if (!c) return fail(TPB200_ERR_CUDA, "out of host memory");
    c->n = n_gpus;
    c->g.resize(n_gpus);
    // peer access between every pair of distinct GPUs: the fused exchange stores into peer memory
    bool peers = distinct && n_gpus > 1;
    if (peers) {
        for (int i = 0; i < n_gpus && peers; ++i)
            for (int j = 0; j < n_gpus && peers; ++j) {
                if (i == j) continue;
                int can = 0;
                if (cudaDeviceCanAccessPeer(&can, devices[i], devices[j]) != cudaSuccess || !can) peers = false;
            }
    }
    if (peers) {
        for (int i = 0; i < n_gpus; ++i) {
            cudaSetDevice(devices[i]);
            for (int j = 0; j < n_gpus; ++j) {
                if (i == j) continue;
                const cudaError_t e = cudaDeviceEnablePeerAccess(devices[j], 0);
                if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) peers = false;
                (void)cudaGetLastError();
            }
        }
    }
    c->fused = peers || n_gpus == 1;
    const size_t xbytes = tpb200_exchange_buffer_bytes();
    cudaError_t e = cudaSuccess;
    for (int i = 0; i < n_gpus && e == cudaSuccess; ++i) {
        CommGpu& q = c->g[i];
        q.device = devices[i];
        e = cudaSetDevice(q.device);
        if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&q.stream, cudaStreamNonBlocking);
        if (e == cudaSuccess) e = cudaMalloc(&q.exchange, xbytes);
        if (e == cudaSuccess) e = cudaMemset(q.exchange, 0, xbytes);
        if (e == cudaSuccess) e = cudaMalloc(&q.scratch, kCommScratchBytes);
        if (e == cudaSuccess) e = cudaMalloc((void**)&q.records, (size_t)n_gpus * TPB200_PARTIAL_BYTES);
        if (e == cudaSuccess) e = cudaMalloc((void**)&q.cand_val, (size_t)n_gpus * kCommMaxK * sizeof(float));
        if (e == cudaSuccess) e = cudaMalloc((void**)&q.cand_idx, (size_t)n_gpus * kCommMaxK * sizeof(int64_t));
        if (e == cudaSuccess) e = cudaMalloc((void**)&q.offsets, (size_t)n_gpus * sizeof(int64_t));
        if (e == cudaSuccess) e = cudaMalloc((void**)&q.out_val, kCommMaxK * sizeof(float));
        if (e == cudaSuccess) e = cudaMalloc((void**)&q.out_idx, kCommMaxK * sizeof(int64_t));
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&q.ready, cudaEventDisableTiming);
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&q.gathered, cudaEventDisableTiming);
        if (e == cudaSuccess) e = cudaDeviceSynchronize();
    }
    if (e != cudaSuccess) {
        for (auto& q : c->g) free_gpu(q);
        delete c;
        return cuda_fail(e, "tpb200_comm_create");
    }
    *out = c;
    return TPB200_OK;
}

extern "C" int tpb200_comm_destroy(tpb200_comm* c) {
    if (!c) return TPB200_OK;
    DeviceGuard guard;
    for (auto& q : c->g) free_gpu(q);
    delete c;
    return TPB200_OK;
}

extern "C" int tpb200_comm_size(const tpb200_comm* c) { return c ? c->n : 0; }
extern "C" int tpb200_comm_fused(const tpb200_comm* c) { return c && c->fused ? 1 : 0; }

extern "C" void* tpb200_comm_stream(const tpb200_comm* c, int g) {
    if (!c || g < 0 || g >= c->n) return nullptr;
    return (void*)c->g[g].stream;
}

extern "C" int tpb200_comm_synchronize(tpb200_comm* c) {
    if (!c) return fail(TPB200_ERR_INVALID, "comm is NULL");
    DeviceGuard guard;
    for (auto& q : c->g) {
        TPB_CUDA_OK(cudaSetDevice(q.device));
        TPB_CUDA_OK(cudaStreamSynchronize(q.stream));
    }
    return TPB200_OK;
}

// Copy `bytes` from GPU s (src) into slot memory of GPU d (dst), on d's stream, after s's `ready`.
static cudaError_t gather_copy(tpb200_comm* c, int d, void* dst, int s, const void* src, size_t bytes) {
    CommGpu& D = c->g[d];
    CommGpu& S = c->g[s];
    cudaError_t e = cudaSetDevice(D.device);
    if (e == cudaSuccess && s != d) e = cudaStreamWaitEvent(D.stream, S.ready, 0);
    if (e != cudaSuccess) return e;
    if (D.device == S.device) return cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, D.stream);
    return cudaMemcpyPeerAsync(dst, D.device, src, S.device, bytes, D.stream);
}

extern "C" int tpb200_reduce_sharded(tpb200_comm* c, int op, const void* const* parts, const int64_t* counts,
                                     int dtype, int64_t correction, void* const* out_val, int64_t* const* out_idx) {
    if (!c) return fail(TPB200_ERR_INVALID, "comm is NULL");
    if (!parts || !counts) return fail(TPB200_ERR_INVALID, "parts / counts must not be NULL");
    if (dtype != TPB200_F32) return fail(TPB200_ERR_UNSUPPORTED, "only float32 input is supported (dtype code %d)", dtype);
    const int fam = family_of_op(op);
    if (fam < 0) return fail(TPB200_ERR_UNSUPPORTED, "operator %d has no sharded form", op);
    const int n = c->n;
    int64_t total = 0;
    std::vector<int64_t> offset(n);
    for (int g = 0; g < n; ++g) {
        if (counts[g] < 0) return fail(TPB200_ERR_INVALID, "negative element count for GPU %d", g);
        if (counts[g] > 0 && !parts[g]) return fail(TPB200_ERR_INVALID, "partition %d is NULL", g);
        offset[g] = total;
        total += counts[g];
    }
    const bool wants_val = !(op == TPB200_OP_ARGMAX || op == TPB200_OP_ARGMIN);
    const bool wants_idx = op == TPB200_OP_ARGMAX || op == TPB200_OP_ARGMIN || op == TPB200_OP_MAX_ARGMAX || op == TPB200_OP_MIN_ARGMIN;
    DeviceGuard guard;
    int rc = TPB200_OK;
    if (c->fused) {
        void* peers[kCommMaxGpus];
        for (int g = 0; g < n; ++g) peers[g] = c->g[g].exchange;
        for (int g = 0; g < n; ++g) {
            CommGpu& q = c->g[g];
            TPB_CUDA_OK(cudaSetDevice(q.device));
            void* ov = wants_val ? (out_val && out_val[g] ? out_val[g] : (void*)q.out_val) : nullptr;
            int64_t* oi = wants_idx ? (out_idx && out_idx[g] ? out_idx[g] : q.out_idx) : nullptr;
            rc = tpb200_reduce_fused_exchange(op, parts[g], dtype, counts[g], offset[g], total, correction, g, n, peers,
                                              ov, oi, q.scratch, kCommScratchBytes, q.stream);
            if (rc) return rc;
        }
        return TPB200_OK;
    }
    // gather mode: record per partition, records to every GPU, rank-ordered merge on every GPU
    for (int g = 0; g < n; ++g) {
        CommGpu& q = c->g[g];
        TPB_CUDA_OK(cudaSetDevice(q.device));
        // the slot of rank g in this GPU's own gather buffer is the kernel's output
        rc = tpb200_reduce_partial(fam, parts[g], dtype, counts[g], offset[g], q.records + (size_t)g * TPB200_PARTIAL_BYTES,
                                   q.scratch, kCommScratchBytes, q.stream);
        if (rc) return rc;
        TPB_CHECKED_SERIALIZE(q.stream);
        TPB_CUDA_OK(cudaEventRecord(q.ready, q.stream));
    }
    for (int d = 0; d < n; ++d) {
        for (int s = 0; s < n; ++s) {
            if (s == d) continue;
            const cudaError_t e = gather_copy(c, d, c->g[d].records + (size_t)s * TPB200_PARTIAL_BYTES, s,
                                              c->g[s].records + (size_t)s * TPB200_PARTIAL_BYTES, TPB200_PARTIAL_BYTES);
            if (e != cudaSuccess) return cuda_fail(e, "record gather");
        }
    }
    for (int g = 0; g < n; ++g) {
        CommGpu& q = c->g[g];
        TPB_CUDA_OK(cudaSetDevice(q.device));
        void* ov = wants_val ? (out_val && out_val[g] ? out_val[g] : (void*)q.out_val) : nullptr;
        int64_t* oi = wants_idx ? (out_idx && out_idx[g] ? out_idx[g] : q.out_idx) : nullptr;
        rc = tpb200_reduce_combine(op, q.records, n, total, correction, ov, oi, q.stream);
        if (rc) return rc;
        TPB_CHECKED_SERIALIZE(q.stream);
        // the next call overwrites the gather buffers of the others: they wait for this merge
        TPB_CUDA_OK(cudaEventRecord(q.gathered, q.stream));
    }
    for (int g = 0; g < n; ++g) {
        TPB_CUDA_OK(cudaSetDevice(c->g[g].device));
        for (int d = 0; d < n; ++d)
            if (d != g) TPB_CUDA_OK(cudaStreamWaitEvent(c->g[g].stream, c->g[d].gathered, 0));
    }
    return TPB200_OK;
}

extern "C" int tpb200_topk_sharded(tpb200_comm* c, const void* const* parts, const int64_t* counts, int dtype,
                                   int64_t k, int largest, float* const* out_val, int64_t* const* out_idx) {
    if (!c) return fail(TPB200_ERR_INVALID, "comm is NULL");
    if (!parts || !counts) return fail(TPB200_ERR_INVALID, "parts / counts must not be NULL");
    if (dtype != TPB200_F32) return fail(TPB200_ERR_UNSUPPORTED, "only float32 input is supported (dtype code %d)", dtype);
    const int n = c->n;
    if (k < 1 || k > kCommMaxK || (int64_t)n * k > 8192)
        return fail(TPB200_ERR_UNSUPPORTED, "k must be in 1..%d with GPUs * k <= 8192 (%d GPUs, k = %lld)", kCommMaxK, n, (long long)k);
    std::vector<int64_t> offset(n);
    int64_t total = 0;
    for (int g = 0; g < n; ++g) {
        if (counts[g] < k) return fail(TPB200_ERR_INVALID, "every GPU must hold at least k elements (GPU %d holds %lld)", g, (long long)counts[g]);
        if (!parts[g]) return fail(TPB200_ERR_INVALID, "partition %d is NULL", g);
        offset[g] = total;
        total += counts[g];
    }
    DeviceGuard guard;
    for (int g = 0; g < n; ++g) {
        CommGpu& q = c->g[g];
        TPB_CUDA_OK(cudaSetDevice(q.device));
        const int64_t sizes[1] = {counts[g]}, strides[1] = {1};
        const size_t need = tpb200_topk_workspace_bytes(dtype, 1, sizes, strides, 0, k);
        if (need > kCommScratchBytes) return fail(TPB200_ERR_WORKSPACE, "local top-k needs %zu bytes of scratch, the comm holds %zu", need, kCommScratchBytes);
        int rc = tpb200_topk(parts[g], dtype, 1, sizes, strides, 0, k, largest, 1, q.cand_val + (size_t)g * k,
                             q.cand_idx + (size_t)g * k, q.scratch, kCommScratchBytes, q.stream);
        if (rc) return rc;
        TPB_CHECKED_SERIALIZE(q.stream);
        TPB_CUDA_OK(cudaMemcpyAsync(q.offsets, offset.data(), sizeof(int64_t) * n, cudaMemcpyHostToDevice, q.stream));
        TPB_CUDA_OK(cudaEventRecord(q.ready, q.stream));
    }
    for (int d = 0; d < n; ++d) {
        for (int s = 0; s < n; ++s) {
            if (s == d) continue;
            cudaError_t e = gather_copy(c, d, c->g[d].cand_val + (size_t)s * k, s, c->g[s].cand_val + (size_t)s * k, sizeof(float) * k);
            if (e == cudaSuccess) e = gather_copy(c, d, c->g[d].cand_idx + (size_t)s * k, s, c->g[s].cand_idx + (size_t)s * k, sizeof(int64_t) * k);
            if (e != cudaSuccess) return cuda_fail(e, "candidate gather");
        }
    }
    for (int g = 0; g < n; ++g) {
        CommGpu& q = c->g[g];
        TPB_CUDA_OK(cudaSetDevice(q.device));
        float* ov = out_val && out_val[g] ? out_val[g] : q.out_val;
        int64_t* oi = out_idx && out_idx[g] ? out_idx[g] : q.out_idx;
        int rc = tpb200_topk_merge(q.cand_val, q.cand_idx, (int64_t)n * k, k, largest, q.offsets, k, ov, oi, q.stream);
        if (rc) return rc;
        TPB_CHECKED_SERIALIZE(q.stream);
        TPB_CUDA_OK(cudaEventRecord(q.gathered, q.stream));
    }
    for (int g = 0; g < n; ++g) {
        TPB_CUDA_OK(cudaSetDevice(c->g[g].device));
        for (int d = 0; d < n; ++d)
            if (d != g) TPB_CUDA_OK(cudaStreamWaitEvent(c->g[g].stream, c->g[d].gathered, 0));
    }
    return TPB200_OK;
}

// Result buffers of GPU g for calls that passed no output pointer for it.
extern "C" void* tpb200_comm_result_values(const tpb200_comm* c, int g) { return c && g >= 0 && g < c->n ? (void*)c->g[g].out_val : nullptr; }
extern "C" int64_t* tpb200_comm_result_indices(const tpb200_comm* c, int g) { return c && g >= 0 && g < c->n ? c->g[g].out_idx : nullptr; }
