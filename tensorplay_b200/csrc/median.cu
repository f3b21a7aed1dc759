// median of a whole float32 tensor on sm_100a, behind tpb200_median.
// The reference has a CPU kernel only (p10/src/backend/cpu/ReductionKernels.cpp:874-901: clone,
// std::nth_element, element (n - 1) / 2 -- the lower of the two middle elements for even n) and
// nothing on CUDA.  Here: an exact radix select over order-preserving 32-bit keys, three sweeps
// over the input (11 + 11 + 10 bits), no copy, no sort.
//   key      increasing with the value; -0.0 folded onto +0.0; every NaN becomes the largest key, so
//            NaNs rank after all numbers (the order the top-k contract uses for "smallest first").
//   sweep p  histogram of digit p of the keys whose higher digits equal the prefix found so far
//            (shared-memory histogram per CTA, merged into global memory with one atomic per bin);
//   pick     one CTA scans the 2048 bins, finds the bin that holds the wanted rank, extends the
//            prefix, reduces the rank and clears the bins for the next sweep.
// After the third pick the prefix is the key of the median; its value is written to the output.
// The second sweep also copies the elements that match the first digit (the median's bin of the first
// histogram: a fraction of a percent of ordinary data) into a buffer of 2^20 floats behind the state;
// the third sweep reads that buffer instead of the input when everything fitted, so the input is
// read twice, not three times.  Everything stays on the stream: state and buffer live in the caller's
// workspace.
#define TPB_FILE_ID 5
#include "common.cuh"
#include "host_util.h"

#include <algorithm>

namespace tpb {

constexpr int kMedBins = 2048;
constexpr int kMedThreads = 512;

constexpr unsigned kMedCand = 1u << 20;    // floats kept from the second sweep
constexpr int kMedKeep = 2048;             // of which per CTA, staged in shared memory

struct MedianState {
    unsigned long long rank;      // rank still wanted among the keys that match the prefix
    unsigned prefix;              // digits found so far, right-aligned
    unsigned kept;                // elements the second sweep wanted to keep (may exceed kMedCand: then none are used)
    unsigned hist[kMedBins];
    unsigned pad2[2];
    float cand[kMedCand];
};

__device__ __forceinline__ unsigned median_key(float x) {
    if (x != x) return 0xffffffffu;
    unsigned b = __float_as_uint(x);
    if ((b << 1) == 0u) b = 0u;
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float median_value(unsigned key) {
    if (key == 0xffffffffu) return NAN;
    const unsigned b = (key & 0x80000000u) ? (key & 0x7fffffffu) : ~key;
    return __uint_as_float(b);
}

struct MedGeom {
    int nd;
    long long size[TPB200_MAX_DIMS], stride[TPB200_MAX_DIMS];
};

// shift / bits of digit p, and the number of key bits above it
__device__ __forceinline__ void digit_of_pass(int pass, int* shift, int* bits) {
    *shift = pass == 0 ? 21 : (pass == 1 ? 10 : 0);
    *bits = pass == 2 ? 10 : 11;
}

template <bool CONTIG>
__global__ void __launch_bounds__(kMedThreads)
median_hist_kernel(const float* __restrict__ in, long long n, MedGeom g, int pass, MedianState* st) {
    __shared__ unsigned hist[kMedBins];
    __shared__ float keep[kMedKeep];        // second sweep: this CTA's elements for the last sweep
    __shared__ unsigned keep_n, keep_over, keep_base;
    const int tid = threadIdx.x;
    for (int i = tid; i < kMedBins; i += kMedThreads) hist[i] = 0u;
    if (tid == 0) { keep_n = 0u; keep_over = 0u; keep_base = 0u; }
    __syncthreads();
    int shift, bits;
    digit_of_pass(pass, &shift, &bits);
    const unsigned mask = (1u << bits) - 1u;
    const unsigned prefix = *TPB_CK(&st->prefix);
    const int above = shift + bits;             // key >> above must equal the prefix (pass 0: nothing above)
    auto count = [&](float x) {
        const unsigned key = median_key(x);
        if (pass == 0 || (key >> above) == prefix) {
            // (adding once per group of lanes with the same bin, found with __match_any_sync, was measured:
            //  118 us per call against 51 us -- the match costs more than the conflicts it removes)
            atomicAdd(&hist[(key >> shift) & mask], 1u);
            if (pass == 1 && *(volatile unsigned*)&keep_over == 0u) {
                // kept in shared memory first: one global atomic per CTA at the end.  A CTA that finds more
                // than its buffer holds (heavy ties) gives up keeping, and the last sweep reads the input.
                const unsigned p = atomicAdd(&keep_n, 1u);
                if (p < (unsigned)kMedKeep) keep[p] = x; else *(volatile unsigned*)&keep_over = 1u;
            }
        }
    };
    const long long gtid = (long long)blockIdx.x * kMedThreads + tid, gthreads = (long long)gridDim.x * kMedThreads;
    const unsigned kept = pass == 2 ? *TPB_CK(&st->kept) : 0u;
    if (pass == 2 && kept <= kMedCand) {
        // everything that matches the first digit is in the buffer: the input is not read again
        for (long long i = gtid; i < (long long)kept; i += gthreads) count(*TPB_CK(&st->cand[i]));
    } else if (CONTIG) {
        // 16-byte loads on the aligned body, scalars at both ends
        long long head = (long long)((4 - (((uintptr_t)in >> 2) & 3)) & 3);
        if (head > n) head = n;
        for (long long i = gtid; i < head; i += gthreads) count(ld_stream1(in + i));
        const float* q = in + head;
        const long long nvec = (n - head) >> 2;
        long long i = gtid;
        for (; i + 3 * gthreads < nvec; i += 4 * gthreads) {
            float4 v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) v[u] = ld_stream4(q + ((i + u * gthreads) << 2));
#pragma unroll
            for (int u = 0; u < 4; ++u) { count(v[u].x); count(v[u].y); count(v[u].z); count(v[u].w); }
        }
        for (; i < nvec; i += gthreads) {
            const float4 v = ld_stream4(q + (i << 2));
            count(v.x); count(v.y); count(v.z); count(v.w);
        }
        for (long long j = head + (nvec << 2) + gtid; j < n; j += gthreads) count(ld_stream1(in + j));
    } else {
        for (long long i = gtid; i < n; i += gthreads) {
            long long off = 0, q = i;
            for (int d = g.nd - 1; d >= 0; --d) {
                const long long c = q % g.size[d];
                q /= g.size[d];
                off += c * g.stride[d];
            }
            count(ld_stream1(in + off));
        }
    }
    __syncthreads();
    for (int i = tid; i < kMedBins; i += kMedThreads) {
        const unsigned c = hist[i];
        if (c) atomicAdd(TPB_CK(&st->hist[i]), c);
    }
    if (pass == 1) {
        const unsigned mine = keep_over ? 0u : keep_n;
        if (tid == 0) keep_base = atomicAdd(TPB_CK(&st->kept), keep_over ? kMedCand + 1u : mine);   // an overflow spoils the buffer for everybody
        __syncthreads();
        const unsigned base = keep_base;
        for (unsigned i = tid; i < mine; i += kMedThreads)
            if (base + i < kMedCand) *TPB_CK(&st->cand[base + i]) = keep[i];
    }
}

// One CTA: which bin holds the wanted rank?  Bins are in ascending key order.
__global__ void __launch_bounds__(1024)
median_pick_kernel(MedianState* st, int pass, float* out) {
    __shared__ unsigned long long wsum[32];
    __shared__ int found;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    // 2048 bins over 1024 threads: two adjacent bins each
    const unsigned long long c0 = *TPB_CK(&st->hist[2 * tid]), c1 = *TPB_CK(&st->hist[2 * tid + 1]);
    unsigned long long incl = c0 + c1;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const unsigned long long t = __shfl_up_sync(kFull, incl, d);
        if (lane >= d) incl += t;
    }
    if (lane == 31) wsum[warp] = incl;
    if (tid == 0) found = -1;
    __syncthreads();
    unsigned long long before = 0;
    for (int w = 0; w < warp; ++w) before += wsum[w];
    const unsigned long long excl = before + incl - (c0 + c1);   // keys in the bins below 2 * tid
    const unsigned long long rank = *TPB_CK(&st->rank);
    __syncthreads();
    if (rank >= excl && rank < excl + c0) found = 2 * tid;
    else if (rank >= excl + c0 && rank < excl + c0 + c1) found = 2 * tid + 1;
    __syncthreads();
    const int bin = found;
    *TPB_CK(&st->hist[2 * tid]) = 0u;          // clean for the next sweep (and the next call)
    *TPB_CK(&st->hist[2 * tid + 1]) = 0u;
    if (bin >= 0 && (bin >> 1) == tid) {
        const int bits = pass == 2 ? 10 : 11;
        const unsigned prefix = pass == 0 ? (unsigned)bin : ((*TPB_CK(&st->prefix) << bits) | (unsigned)bin);
        *TPB_CK(&st->prefix) = prefix;
        *TPB_CK(&st->rank) = rank - (excl + ((bin & 1) ? c0 : 0ull));
        if (pass == 2) *TPB_CK(&out[0]) = median_value(prefix);
    }
}

__global__ void median_init_kernel(MedianState* st, unsigned long long rank, float* out, int empty) {
    const int tid = threadIdx.x;
    for (int i = tid; i < kMedBins; i += blockDim.x) *TPB_CK(&st->hist[i]) = 0u;
    if (tid == 0) {
        *TPB_CK(&st->rank) = rank;
        *TPB_CK(&st->prefix) = 0u;
        *TPB_CK(&st->kept) = 0u;
        if (empty) *TPB_CK(&out[0]) = NAN;   // the reference returns NaN for an empty tensor (ReductionKernels.cpp:877)
    }
}

}  // namespace tpb

using namespace tpb;

extern "C" size_t tpb200_median_workspace_bytes(void) { return sizeof(MedianState); }

extern "C" int tpb200_median(const void* in, int dtype, int ndim, const int64_t* sizes, const int64_t* strides,
                             void* out, void* workspace, size_t workspace_bytes, void* stream) {
    if (dtype != TPB200_F32) return fail(TPB200_ERR_UNSUPPORTED, "only float32 input is supported (dtype code %d)", dtype);
    if (ndim < 0 || ndim > TPB200_MAX_DIMS) return fail(TPB200_ERR_UNSUPPORTED, "tensors of rank %d are not supported (max %d)", ndim, TPB200_MAX_DIMS);
    if (ndim > 0 && (!sizes || !strides)) return fail(TPB200_ERR_INVALID, "sizes/strides must not be NULL");
    if (!out) return fail(TPB200_ERR_INVALID, "out is NULL");
    if (!workspace || workspace_bytes < sizeof(MedianState))
        return fail(TPB200_ERR_WORKSPACE, "workspace of %zu bytes required, %zu given", sizeof(MedianState), workspace ? workspace_bytes : (size_t)0);
    if (((uintptr_t)workspace) & 7) return fail(TPB200_ERR_WORKSPACE, "workspace must be 8-byte aligned");
    long long n = 1;
    MedGeom g{};
    bool contig = true;
    {
        // drop size-1 dims; contiguous if the rest has row-major strides
        for (int i = 0; i < ndim; ++i) {
            if (sizes[i] < 0) return fail(TPB200_ERR_INVALID, "negative size in dim %d", i);
            n *= sizes[i];
            if (sizes[i] == 1) continue;
            g.size[g.nd] = sizes[i];
            g.stride[g.nd] = strides[i];
            ++g.nd;
        }
        long long acc = 1;
        for (int i = g.nd - 1; i >= 0; --i) {
            if (g.stride[i] != acc) contig = false;
            acc *= g.size[i];
        }
    }
    if (n > 0 && !in) return fail(TPB200_ERR_INVALID, "input pointer is NULL");
    cudaStream_t st = (cudaStream_t)stream;
    TPB_CHECK_RANGES(st, view_range(in, ndim, sizes, strides, 4), HostRange{out, 4}, HostRange{workspace, sizeof(MedianState)});
    MedianState* state = (MedianState*)workspace;
    float* o = (float*)out;
    const unsigned long long rank = n > 0 ? (unsigned long long)((n - 1) / 2) : 0ull;
    TPB_LAUNCH("median_init_kernel", median_init_kernel, dim3(1), 256, 0, st, state, rank, o, n == 0 ? 1 : 0);
    if (n == 0) return TPB200_OK;
    const int sms = sm_count();
    const long long want = ceil_div(n, (long long)kMedThreads * 16);
    const dim3 grid((unsigned)std::max(1LL, std::min<long long>(want, (long long)sms * 4)));
    for (int pass = 0; pass < 3; ++pass) {
        if (contig) TPB_LAUNCH("median_hist_kernel", median_hist_kernel<true>, grid, kMedThreads, 0, st, (const float*)in, n, g, pass, state);
        else        TPB_LAUNCH("median_hist_kernel", median_hist_kernel<false>, grid, kMedThreads, 0, st, (const float*)in, n, g, pass, state);
        TPB_LAUNCH("median_pick_kernel", median_pick_kernel, dim3(1), 1024, 0, st, state, pass, o);
    }
    return TPB200_OK;
}
