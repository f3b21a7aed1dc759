// top-k along one dim for float32 tensors on sm_100a, behind tpb200_topk / tpb200_topk_merge.
// The reference has no top-k kernel; the contract is the one stated in include/tpb200.h:
// first k entries of the row stably sorted by value, ties in ascending index (the tie rule of
// the reference's argmax scan, p10/src/backend/cpu/ReductionKernels.cpp:727-735).
//
// Order.  Every element gets a 64-bit rank word  (key << 32) | (0xFFFFFFFF - index)  where key is
// the order-preserving float->uint32 transform (flipped for smallest-first; -0.0 folded onto
// +0.0; NaN -> 0).  Larger word = earlier in the output.  All words of a row are distinct, so
// "top k by rank word" IS the stable order including its tie rule -- no separate tie pass.
//
// One HBM pass.  A row (or a fixed slice of it) is streamed once by one CTA in tiles of
// 512 threads x 4 x float4.  The CTA keeps a candidate buffer of rank words in shared memory
// and an exclusive threshold tau: an element is a candidate iff its word > tau.  On the hot
// path that test is ONE float compare per element (x > value(tau)): within a CTA indices only
// grow, so an element equal to the threshold value always loses its tie.  tau starts from the
// k-th largest of per-thread group maxima of the first tile (a valid lower bound of the k-th
// best) and rises every time the buffer fills and is cut back to its k best (bitonic sort in
// shared memory).  Rows shorter than a few tiles are sorted whole in shared memory instead;
// rows split over several CTAs are merged by a second, tiny kernel.
#include "common.cuh"
#include "host_util.h"

#include <algorithm>
#include <mutex>
#include <string>

namespace tpb {

constexpr int kStreamThreads = 256;
constexpr int kTile = kStreamThreads * 16;                    // 4096 elements = one 16 KB stage
constexpr int kStages = 4;                                    // shared-memory ring depth
constexpr int kSortThreads = 512;
constexpr int kMaxStreamK = 2048;                             // largest k of the streaming path
constexpr int kMaxSortRow = 16384;                            // longest row sorted whole in smem
constexpr int kMaxMergeCand = 8192;                           // tpb200_topk_merge limit

// ------------------------------------------------------------------ rank words -------------
template <bool LARGEST>
__device__ __forceinline__ unsigned rank_key(float x) {
    if (x != x) return 0u;
    unsigned b = __float_as_uint(x);
    if ((b << 1) == 0u) b = 0u;  // -0.0 ties with +0.0
    b = (b & 0x80000000u) ? ~b : (b | 0x80000000u);
    return LARGEST ? b : ~b;
}
template <bool LARGEST>
__device__ __forceinline__ float key_value(unsigned key) {
    unsigned b = LARGEST ? key : ~key;
    b = (b & 0x80000000u) ? (b & 0x7fffffffu) : ~b;
    return __uint_as_float(b);
}
template <bool LARGEST>
__device__ __forceinline__ unsigned long long rank_word(float x, unsigned idx) {
    return ((unsigned long long)rank_key<LARGEST>(x) << 32) | (unsigned long long)(0xffffffffu - idx);
}
__device__ __forceinline__ unsigned word_index(unsigned long long w) { return 0xffffffffu - (unsigned)w; }

// Descending bitonic sort of a[0..n), n a power of two, by all threads of the CTA.
__device__ void bitonic_desc(unsigned long long* a, int n, int tid, int nthr) {
    for (int size = 2; size <= n; size <<= 1) {
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            for (int t = tid; t < (n >> 1); t += nthr) {
                int lo = ((t & ~(stride - 1)) << 1) | (t & (stride - 1));
                int hi = lo | stride;
                bool desc = (lo & size) == 0;
                unsigned long long x = a[lo], y = a[hi];
                if ((x < y) == desc) { a[lo] = y; a[hi] = x; }
            }
            __syncthreads();
        }
    }
}

// ------------------------------------------------------------------ geometry ---------------
struct TopkGeom {
    long long rows;       // independent rows
    long long k1;         // rows = k0 * k1 (two kept dims at most)
    long long ks0, ks1;   // their strides
    long long len;        // row length
    long long es;         // element stride along the row
    long long k;
    long long chunk;      // slice length per CTA
    int S;                // slices per row
    int B;                // candidate buffer capacity (power of two)
    int soft;             // buffer fill that triggers a cut at the next tile boundary
};

__device__ __forceinline__ const float* topk_row(const float* in, const TopkGeom& g, long long r) {
    long long a = r / g.k1;
    long long b = r - a * g.k1;
    return in + a * g.ks0 + b * g.ks1;
}

// ------------------------------------------------------------------ streaming kernel -------
// Shared-memory ring: kStages tiles of kTile floats, filled by cp.async.bulk (one elected thread
// issues, an mbarrier per stage counts the bytes), consumed by all 256 threads.  The CTA-wide
// barrier that ends every tile also tells the issuing thread that the stage may be refilled, so
// up to (kStages-1) x 16 KB are in flight per CTA while a tile is being compared.
struct StreamShared {
    unsigned long long full[kStages];
    unsigned long long tau;
    int cnt;
    int err;
};

template <bool LARGEST>
__device__ __forceinline__ float worst_value() { return LARGEST ? -INFINITY : INFINITY; }

// Register path for rows that cannot use bulk copies (element stride != 1, or not 16-byte
// aligned): this thread's 16 elements of the tile; absent ones get the worst value.
template <bool LARGEST>
__device__ __forceinline__ void load_tile_direct(float (&x)[16], const float* slice, long long es,
                                                 long long len, long long tile_off, int tid) {
#pragma unroll
    for (int u = 0; u < 4; ++u) {
        long long e0 = tile_off + ((long long)u * kStreamThreads + tid) * 4;
#pragma unroll
        for (int c = 0; c < 4; ++c)
            x[4 * u + c] = (e0 + c < len) ? ld_stream1(slice + (e0 + c) * es) : worst_value<LARGEST>();
    }
}

// Cut the buffer back to its k best: zero-fill to a power of two, sort descending, publish the
// new count and threshold.  Entered by every thread after a barrier that made all appends visible.
__device__ void compact(unsigned long long* buf, StreamShared* sh, int B, int k, int tid, int nthr) {
    int n = sh->cnt;
    if (n > B) n = B;
    int N = 2;
    while (N < n) N <<= 1;
    for (int i = n + tid; i < N; i += nthr) buf[i] = 0ull;
    __syncthreads();
    bitonic_desc(buf, N, tid, nthr);
    if (tid == 0) {
        sh->cnt = n < k ? n : k;
        sh->tau = n >= k ? buf[k - 1] : 0ull;
    }
    __syncthreads();
}

template <bool LARGEST, bool BULK>
__global__ void __launch_bounds__(kStreamThreads, 3)
topk_stream_kernel(const float* __restrict__ in, TopkGeom g, unsigned long long* __restrict__ ws,
                   float* __restrict__ out_val, long long* __restrict__ out_idx, int* status) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    float* ring = reinterpret_cast<float*>(smem_raw);
    unsigned long long* buf =
        reinterpret_cast<unsigned long long*>(smem_raw + (BULK ? (size_t)kStages * kTile * sizeof(float) : 0));
    __shared__ StreamShared sh;
    const int tid = threadIdx.x, lane = tid & 31;
    const int s = blockIdx.x;
    const long long r = blockIdx.y;
    const float* row = topk_row(in, g, r);
    const long long begin = (long long)s * g.chunk;
    long long len = g.len - begin;
    if (len > g.chunk) len = g.chunk;
    const float* slice = row + begin * g.es;
    const int ntiles = (int)((len + kTile - 1) / kTile);
    const int B = g.B, k = (int)g.k, soft_limit = g.soft;

    // thread 0: start the copy of tile u into its stage (a ragged tail of < 4 floats by hand)
    auto issue = [&](int u) {
        const int st = u % kStages;
        const long long off = (long long)u * kTile;
        long long n = len - off;
        if (n > kTile) n = kTile;
        const int n4 = (int)(n & ~3LL);
        float* dst = ring + (size_t)st * kTile;
        for (int i = n4; i < (int)n; ++i) dst[i] = ld_stream1(slice + off + i);
        if (n4 > 0) {
            mbar_arrive_expect_tx(&sh.full[st], (unsigned)n4 * 4u);
            bulk_g2s(dst, slice + off, (unsigned)n4 * 4u, &sh.full[st]);
        } else {
            mbar_arrive(&sh.full[st]);
        }
    };

    if (tid == 0) {
        sh.cnt = 0; sh.tau = 0ull; sh.err = 0;
        if (BULK) {
            for (int i = 0; i < kStages; ++i) mbar_init(&sh.full[i], 1);
            fence_mbar_init();
        }
    }
    __syncthreads();
    if (BULK && tid == 0)
        for (int u = 0; u < kStages && u < ntiles; ++u) issue(u);

    unsigned long long tau = 0ull;  // exclusive: candidate iff word > tau
    float tvf = worst_value<LARGEST>();
    int mode = 0;                   // 0 accept everything, 1 float compare, 2 integer compare

    for (int t = 0; t < ntiles; ++t) {
        const long long tile_off = (long long)t * kTile;
        float x[16];
        bool timeout = false;
        if (BULK) {
            const int st = t % kStages;
            timeout = !mbar_wait_bounded(&sh.full[st], (unsigned)((t / kStages) & 1));
            const float4* src = reinterpret_cast<const float4*>(ring + (size_t)st * kTile);
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                float4 v = src[u * kStreamThreads + tid];
                x[4 * u] = v.x; x[4 * u + 1] = v.y; x[4 * u + 2] = v.z; x[4 * u + 3] = v.w;
            }
        } else {
            load_tile_direct<LARGEST>(x, slice, g.es, len, tile_off, tid);
        }

        // position of x[4u+c] in the row: begin + tile_off + (u*256 + tid)*4 + c
        unsigned valid = 0xffffu;
        if (tile_off + kTile > len) {
            valid = 0u;
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                long long e = tile_off + ((long long)(j >> 2) * kStreamThreads + tid) * 4 + (j & 3);
                if (e < len) valid |= 1u << j;
                else x[j] = worst_value<LARGEST>();
            }
        }
        auto idx_of = [&](int j) -> unsigned {
            return (unsigned)(begin + tile_off + ((long long)(j >> 2) * kStreamThreads + tid) * 4 + (j & 3));
        };

        unsigned m = 0u;
        if (mode == 1) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                bool p = LARGEST ? (x[j] > tvf) : (x[j] < tvf);
                m |= p ? (1u << j) : 0u;
            }
        } else if (mode == 0 && t == 0 && len >= kTile && k <= kStreamThreads) {
            // bootstrap: the k-th largest of the 256 per-thread maxima bounds the k-th best from below
            unsigned long long gm = 0ull;
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                unsigned long long w = rank_word<LARGEST>(x[j], idx_of(j));
                gm = w > gm ? w : gm;
            }
            buf[tid] = gm;
            __syncthreads();
            bitonic_desc(buf, kStreamThreads, tid, kStreamThreads);
            tau = buf[k - 1] - 1ull;
            __syncthreads();
#pragma unroll
            for (int j = 0; j < 16; ++j)
                m |= (rank_word<LARGEST>(x[j], idx_of(j)) > tau) ? (1u << j) : 0u;
            // later tiles hold larger indices than the threshold element, so there "word > tau"
            // is "key > key(tau)", one float compare (tau's low word is never 0, so the -1 above
            // did not borrow from the key)
            mode = (tau >> 32) == 0ull ? 2 : 1;
            tvf = key_value<LARGEST>((unsigned)(tau >> 32));
        } else if (mode == 0) {
            m = valid;
        } else {
#pragma unroll
            for (int j = 0; j < 16; ++j)
                m |= (rank_word<LARGEST>(x[j], idx_of(j)) > tau) ? (1u << j) : 0u;
            m &= valid;
        }

        // optimistic append: slots are reserved with one atomic per warp; what does not fit stays
        // pending and forces a cut of the buffer below
        unsigned pending = m;
        auto try_append = [&]() {
            int n = __popc(pending);
            int incl = n;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                int o = __shfl_up_sync(kFull, incl, d);
                if (lane >= d) incl += o;
            }
            int total = __shfl_sync(kFull, incl, 31);
            int base = 0;
            if (lane == 31) base = atomicAdd(&sh.cnt, total);
            base = __shfl_sync(kFull, base, 31);
            int pos = base + incl - n;
            if (pending) {
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    if (pending & (1u << j)) {
                        if (pos < B) {
                            buf[pos] = rank_word<LARGEST>(x[j], idx_of(j));
                            pending &= ~(1u << j);
                        }
                        ++pos;
                    }
                }
            }
        };
        if (__any_sync(kFull, pending != 0u)) try_append();

        const bool soft = tid == 0 && *(volatile int*)&sh.cnt > soft_limit;
        if (__syncthreads_or((pending != 0u) | soft | timeout)) {
            if (timeout) sh.err = 1;
            __syncthreads();
            if (sh.err) {
                // a copy never landed: give the copies still in flight a bounded chance to finish,
                // flag the failure for the host, and leave without touching the outputs
                if (BULK)
                    for (int u = t; u < ntiles && u < t + kStages; ++u)
                        mbar_wait_bounded(&sh.full[u % kStages], (unsigned)((u / kStages) & 1));
                if (tid == 0 && status) atomicExch(status, 1);
                return;
            }
            while (true) {
                compact(buf, &sh, B, k, tid, kStreamThreads);
                tau = sh.tau;
                if (pending) {
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        if ((pending & (1u << j)) && !(rank_word<LARGEST>(x[j], idx_of(j)) > tau))
                            pending &= ~(1u << j);
                }
                if (__any_sync(kFull, pending != 0u)) try_append();
                if (!__syncthreads_or(pending != 0u)) break;
            }
            mode = tau == 0ull ? 0 : ((tau >> 32) == 0ull ? 2 : 1);
            tvf = key_value<LARGEST>((unsigned)(tau >> 32));
        }
        // every thread has its tile in registers: the stage can take tile t + kStages
        if (BULK && tid == 0 && t + kStages < ntiles) issue(t + kStages);
    }

    // final cut: the slice's best min(cnt, k), sorted
    __syncthreads();
    compact(buf, &sh, B, k, tid, kStreamThreads);
    const int cnt = sh.cnt;
    if (ws) {
        unsigned long long* dst = ws + ((size_t)r * g.S + s) * (size_t)k;
        for (int j = tid; j < k; j += kStreamThreads) dst[j] = j < cnt ? buf[j] : 0ull;
    } else {
        for (int j = tid; j < k && j < cnt; j += kStreamThreads) {
            unsigned idx = word_index(buf[j]);
            out_idx[r * k + j] = (long long)idx;
            out_val[r * k + j] = row[(long long)idx * g.es];
        }
    }
}

// ------------------------------------------------------------------ sort kernels -----------
// FROM_ROW: rank every element of a short row.  Otherwise: merge the S*k slice survivors of a row.
// One CTA per row, whole working set in shared memory.
template <bool LARGEST, bool FROM_ROW>
__global__ void __launch_bounds__(kSortThreads)
topk_sort_kernel(const float* __restrict__ in, TopkGeom g, const unsigned long long* __restrict__ ws,
                 int n_items, int N, float* __restrict__ out_val, long long* __restrict__ out_idx) {
    extern __shared__ __align__(16) unsigned long long buf[];
    const int tid = threadIdx.x, nthr = blockDim.x;
    const long long r = blockIdx.x;
    const float* row = topk_row(in, g, r);
    if (FROM_ROW) {
        for (int i = tid; i < N; i += nthr)
            buf[i] = i < n_items ? rank_word<LARGEST>(ld_stream1(row + (long long)i * g.es), (unsigned)i) : 0ull;
    } else {
        const unsigned long long* src = ws + (size_t)r * n_items;
        for (int i = tid; i < N; i += nthr) buf[i] = i < n_items ? src[i] : 0ull;
    }
    __syncthreads();
    bitonic_desc(buf, N, tid, nthr);
    const int k = (int)g.k;
    for (int j = tid; j < k; j += nthr) {
        unsigned idx = word_index(buf[j]);
        out_idx[r * k + j] = (long long)idx;
        out_val[r * k + j] = row[(long long)idx * g.es];
    }
}

// ------------------------------------------------------------------ global merge -----------
// Candidates carry 64-bit tensor-global indices, so the order is on (key, index) pairs.
template <bool LARGEST>
__global__ void __launch_bounds__(kSortThreads)
topk_merge_pairs_kernel(const float* __restrict__ cv, const long long* __restrict__ ci, int n, int N,
                        int k, const long long* __restrict__ list_off, int list_len,
                        float* __restrict__ out_val, long long* __restrict__ out_idx) {
    extern __shared__ __align__(16) unsigned char raw[];
    long long* sidx = reinterpret_cast<long long*>(raw);
    unsigned* skey = reinterpret_cast<unsigned*>(sidx + N);
    int* sslot = reinterpret_cast<int*>(skey + N);
    const int tid = threadIdx.x, nthr = blockDim.x;
    for (int i = tid; i < N; i += nthr) {
        if (i < n) {
            skey[i] = rank_key<LARGEST>(cv[i]);
            sidx[i] = ci[i] + (list_off ? list_off[i / list_len] : 0LL);
            sslot[i] = i;
        }
        else { skey[i] = 0u; sidx[i] = kNoIndex; sslot[i] = -1; }
    }
    __syncthreads();
    for (int size = 2; size <= N; size <<= 1) {
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            for (int t = tid; t < (N >> 1); t += nthr) {
                int lo = ((t & ~(stride - 1)) << 1) | (t & (stride - 1));
                int hi = lo | stride;
                bool desc = (lo & size) == 0;
                unsigned ka = skey[lo], kb = skey[hi];
                long long ia = sidx[lo], ib = sidx[hi];
                // "lo ranks after hi": padding (slot -1) ranks after everything, NaN included
                int sa = sslot[lo], sb = sslot[hi];
                bool a_after_b = (sa < 0) != (sb < 0) ? (sa < 0) : (ka < kb || (ka == kb && ia > ib));
                bool b_after_a = (sa < 0) != (sb < 0) ? (sb < 0) : (kb < ka || (ka == kb && ib > ia));
                if (desc ? a_after_b : b_after_a) {
                    skey[lo] = kb; skey[hi] = ka;
                    sidx[lo] = ib; sidx[hi] = ia;
                    sslot[lo] = sb; sslot[hi] = sa;
                }
            }
            __syncthreads();
        }
    }
    for (int j = tid; j < k; j += nthr) {
        out_idx[j] = sidx[j];
        out_val[j] = cv[sslot[j]];
    }
}

// ------------------------------------------------------------------ device status ----------
// Set to 1 by a kernel whose bounded wait on a bulk copy gave up (its outputs are then not
// written).  One word per device, lives in the module's global memory.
__device__ int g_device_status = 0;

static int* device_status_word() {
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

// ------------------------------------------------------------------ planner ----------------
enum TopkPath { TK_NONE, TK_SORTROW, TK_STREAM };

struct TopkPlan {
    TopkPath path = TK_NONE;
    TopkGeom g{};
    bool vec = false;
    int N = 0;            // sort size of the sort-row path
    int mergeN = 0;       // sort size of the slice merge (S > 1)
    size_t ws_bytes = 0;
    long long out_numel = 0;
};

static int topk_plan(const void* in, int ndim, const int64_t* sizes, const int64_t* strides, int dim,
                     int64_t k, TopkPlan* pl) {
    if (ndim < 0 || ndim > TPB200_MAX_DIMS)
        return fail(TPB200_ERR_UNSUPPORTED, "tensors of rank %d are not supported (max %d)", ndim, TPB200_MAX_DIMS);
    if (ndim > 0 && (!sizes || !strides)) return fail(TPB200_ERR_INVALID, "sizes/strides must not be NULL");
    long long len = 1, es = 1;
    int d = dim;
    if (ndim == 0) {
        if (dim != 0 && dim != -1) return fail(TPB200_ERR_DIM_RANGE, "Dimension out of range");
    } else {
        if (d < 0) d += ndim;
        if (d < 0 || d >= ndim) return fail(TPB200_ERR_DIM_RANGE, "Dimension out of range");
        len = sizes[d];
        es = strides[d];
    }
    if (k < 0 || k > len) return fail(TPB200_ERR_INVALID, "selected index k out of range");
    if (len >= 0xffffffffLL) return fail(TPB200_ERR_UNSUPPORTED, "rows of 2^32-1 or more elements are not supported");

    // kept dims, merged where the strides allow; at most two survive
    struct KD { long long size, stride; };
    KD kept[TPB200_MAX_DIMS];
    int nk = 0;
    long long rows = 1;
    for (int i = 0; i < ndim; ++i) {
        if (i == d) continue;
        if (sizes[i] < 0) return fail(TPB200_ERR_INVALID, "negative size in dim %d", i);
        rows *= sizes[i];
        if (sizes[i] == 1) continue;
        if (nk > 0 && kept[nk - 1].stride == strides[i] * sizes[i]) {
            kept[nk - 1].size *= sizes[i];
            kept[nk - 1].stride = strides[i];
        } else {
            kept[nk].size = sizes[i];
            kept[nk].stride = strides[i];
            ++nk;
        }
    }
    pl->out_numel = rows * k;
    if (rows == 0 || k == 0) { pl->path = TK_NONE; return TPB200_OK; }
    if (nk > 2) return fail(TPB200_ERR_UNSUPPORTED, "top-k needs the non-selected dims to collapse to at most two strided dims");

    TopkGeom& g = pl->g;
    g.rows = rows;
    g.len = len;
    g.es = es;
    g.k = k;
    if (nk == 2) { g.k1 = kept[1].size; g.ks0 = kept[0].stride; g.ks1 = kept[1].stride; }
    else if (nk == 1) { g.k1 = 1; g.ks0 = kept[0].stride; g.ks1 = 0; }
    else { g.k1 = 1; g.ks0 = 0; g.ks1 = 0; }
    g.S = 1;
    g.chunk = len;
    pl->vec = es == 1 && (((uintptr_t)in) & 15) == 0 && g.ks0 % 4 == 0 && g.ks1 % 4 == 0;

    const char* force = getenv("TPB200_FORCE_TOPK");  // "sort" | "stream": experiments only
    const bool force_sort = force && std::string(force) == "sort";
    const bool force_stream = force && std::string(force) == "stream";

    if ((len <= 4096 && !force_stream) || k > kMaxStreamK || (force_sort && len <= kMaxSortRow)) {
        if (len > kMaxSortRow)
            return fail(TPB200_ERR_UNSUPPORTED, "k > %d is only supported on rows of at most %d elements", kMaxStreamK, kMaxSortRow);
        pl->path = TK_SORTROW;
        pl->N = std::max(2, pow2_ceil(len));
        return TPB200_OK;
    }
    if (rows > 65535) {
        // grid.y limit; such shapes have short rows in practice
        return fail(TPB200_ERR_UNSUPPORTED, "more than 65535 rows of more than 4096 elements are not supported");
    }
    pl->path = TK_STREAM;
    g.B = pow2_ceil(std::max<long long>(4 * k, 1024));
    g.soft = (int)std::max<long long>(2 * k, 256);
    // slices: enough CTAs to fill the GPU, each slice at least eight tiles and at least 8k long
    const int sms = sm_count();
    long long want = ceil_div((long long)sms * 4, rows);
    long long most = std::max(1LL, len / std::max<long long>(8 * kTile, 8 * k));
    long long cap = std::max(1LL, (long long)kMaxSortRow / k);
    long long S = std::max(1LL, std::min(std::min(want, most), cap));
    const char* fs = getenv("TPB200_TOPK_SLICES");
    if (fs) S = std::max(1LL, std::min((long long)atoi(fs), cap));
    g.chunk = round_up(ceil_div(len, S), 4);
    g.S = (int)ceil_div(len, g.chunk);
    if (g.S > 1) {
        pl->mergeN = std::max(2, pow2_ceil((long long)g.S * k));
        pl->ws_bytes = (size_t)rows * g.S * k * sizeof(unsigned long long);
    }
    return TPB200_OK;
}

template <class K>
static int allow_smem(K kernel, size_t bytes) {
    if (bytes > 48 * 1024) {
        TPB_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
    }
    return TPB200_OK;
}

template <bool LARGEST>
static int topk_launch(const TopkPlan& pl, const float* in, float* ov, long long* oi, void* ws,
                       cudaStream_t st) {
    const TopkGeom& g = pl.g;
    if (pl.path == TK_SORTROW) {
        size_t sm = (size_t)pl.N * 8;
        int rc = allow_smem(topk_sort_kernel<LARGEST, true>, sm);
        if (rc) return rc;
        int threads = std::min(kSortThreads, std::max(32, pl.N / 2));
        if (g.rows > 0x7fffffffLL) return fail(TPB200_ERR_UNSUPPORTED, "too many rows for one launch");
        topk_sort_kernel<LARGEST, true><<<(unsigned)g.rows, threads, sm, st>>>(in, g, nullptr, (int)g.len, pl.N, ov, oi);
        TPB_LAUNCH_OK("topk_sort_kernel");
        return TPB200_OK;
    }
    dim3 grid((unsigned)g.S, (unsigned)g.rows);
    unsigned long long* w = g.S > 1 ? (unsigned long long*)ws : nullptr;
    int* status = device_status_word();
    if (pl.vec) {
        size_t sm = (size_t)g.B * 8 + (size_t)kStages * kTile * sizeof(float);
        int rc = allow_smem(topk_stream_kernel<LARGEST, true>, sm);
        if (rc) return rc;
        topk_stream_kernel<LARGEST, true><<<grid, kStreamThreads, sm, st>>>(in, g, w, ov, oi, status);
    } else {
        size_t sm = (size_t)g.B * 8;
        int rc = allow_smem(topk_stream_kernel<LARGEST, false>, sm);
        if (rc) return rc;
        topk_stream_kernel<LARGEST, false><<<grid, kStreamThreads, sm, st>>>(in, g, w, ov, oi, status);
    }
    TPB_LAUNCH_OK("topk_stream_kernel");
    if (g.S > 1) {
        size_t msm = (size_t)pl.mergeN * 8;
        int rc = allow_smem(topk_sort_kernel<LARGEST, false>, msm);
        if (rc) return rc;
        int threads = std::min(kSortThreads, std::max(32, pl.mergeN / 2));
        topk_sort_kernel<LARGEST, false><<<(unsigned)g.rows, threads, msm, st>>>(in, g, w, g.S * (int)g.k, pl.mergeN, ov, oi);
        TPB_LAUNCH_OK("topk_sort_kernel(merge)");
    }
    return TPB200_OK;
}

}  // namespace tpb

using namespace tpb;

extern "C" size_t tpb200_topk_workspace_bytes(int dtype, int ndim, const int64_t* sizes,
                                              const int64_t* strides, int dim, int64_t k) {
    if (dtype != TPB200_F32) return 0;
    TopkPlan pl;
    if (topk_plan((const void*)16, ndim, sizes, strides, dim, k, &pl) != TPB200_OK) return 0;
    return pl.ws_bytes;
}

extern "C" int tpb200_topk(const void* in, int dtype, int ndim, const int64_t* sizes,
                           const int64_t* strides, int dim, int64_t k, int largest, int sorted,
                           void* out_val, int64_t* out_idx, void* workspace, size_t workspace_bytes,
                           void* stream) {
    (void)sorted;  // the result is always sorted, which satisfies sorted = 0 as well
    if (dtype != TPB200_F32) return fail(TPB200_ERR_UNSUPPORTED, "only float32 input is supported (dtype code %d)", dtype);
    TopkPlan pl;
    int rc = topk_plan(in, ndim, sizes, strides, dim, k, &pl);
    if (rc) return rc;
    if (pl.path == TK_NONE) return TPB200_OK;
    if (!in) return fail(TPB200_ERR_INVALID, "input pointer is NULL");
    if (!out_val || !out_idx) return fail(TPB200_ERR_INVALID, "out_val / out_idx must not be NULL");
    if (pl.ws_bytes) {
        if (!workspace || workspace_bytes < pl.ws_bytes)
            return fail(TPB200_ERR_WORKSPACE, "workspace of %zu bytes required, %zu given", pl.ws_bytes, workspace ? workspace_bytes : (size_t)0);
        if (((uintptr_t)workspace) & 7) return fail(TPB200_ERR_WORKSPACE, "workspace must be 8-byte aligned");
    }
    cudaStream_t st = (cudaStream_t)stream;
    if (largest) return topk_launch<true>(pl, (const float*)in, (float*)out_val, (long long*)out_idx, workspace, st);
    return topk_launch<false>(pl, (const float*)in, (float*)out_val, (long long*)out_idx, workspace, st);
}

extern "C" int tpb200_topk_merge(const float* cand_val, const int64_t* cand_idx, int64_t n_cand,
                                 int64_t k, int largest, const int64_t* list_offsets, int64_t list_len,
                                 float* out_val, int64_t* out_idx, void* stream) {
    if (n_cand < 0 || n_cand > kMaxMergeCand)
        return fail(TPB200_ERR_UNSUPPORTED, "at most %d candidates can be merged, %lld given", kMaxMergeCand, (long long)n_cand);
    if (k < 0 || k > n_cand) return fail(TPB200_ERR_INVALID, "selected index k out of range");
    if (k == 0) return TPB200_OK;
    if (!cand_val || !cand_idx || !out_val || !out_idx) return fail(TPB200_ERR_INVALID, "NULL pointer argument");
    if (list_offsets && (list_len < 1 || n_cand % list_len != 0))
        return fail(TPB200_ERR_INVALID, "list_len must divide n_cand");
    const long long* lo = (const long long*)list_offsets;
    const int ll = list_offsets ? (int)list_len : 1;
    const int N = std::max(2, pow2_ceil(n_cand));
    const size_t sm = (size_t)N * (8 + 4 + 4);
    cudaStream_t st = (cudaStream_t)stream;
    const int threads = std::min(kSortThreads, std::max(32, N / 2));
    if (largest) {
        int rc = allow_smem(topk_merge_pairs_kernel<true>, sm);
        if (rc) return rc;
        topk_merge_pairs_kernel<true><<<1, threads, sm, st>>>(cand_val, (const long long*)cand_idx, (int)n_cand, N, (int)k, lo, ll, out_val, (long long*)out_idx);
    } else {
        int rc = allow_smem(topk_merge_pairs_kernel<false>, sm);
        if (rc) return rc;
        topk_merge_pairs_kernel<false><<<1, threads, sm, st>>>(cand_val, (const long long*)cand_idx, (int)n_cand, N, (int)k, lo, ll, out_val, (long long*)out_idx);
    }
    TPB_LAUNCH_OK("topk_merge_pairs_kernel");
    return TPB200_OK;
}

extern "C" int tpb200_device_status(int* status_out) {
    if (!status_out) return fail(TPB200_ERR_INVALID, "status_out is NULL");
    int v = 0, zero = 0;
    TPB_CUDA_OK(cudaMemcpyFromSymbol(&v, g_device_status, sizeof(int)));
    if (v != 0) TPB_CUDA_OK(cudaMemcpyToSymbol(g_device_status, &zero, sizeof(int)));
    *status_out = v;
    return TPB200_OK;
}
