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
// One HBM pass.  A row (or a fixed slice of it) is streamed once by one CTA, every warp on its own
// 1024-element tiles.  The CTA keeps candidate rank words in shared memory and an exclusive
// threshold tau: an element is a candidate iff its word > tau.  On the hot path that test is ONE
// float compare per element (x >= value(tau); the exact 64-bit compare is only made for the few
// that pass).  tau starts from the k-th largest of a sample of lane maxima of the first tiles (a
// k-th largest of any subset of the row is a valid lower bound of the k-th best) and rises every
// time candidates are cut back to their k best.  Two streaming kernels share this scheme:
// topk_smallk_kernel (k <= 64: a ring of candidates cut 64 words at a time by single warps, no
// barrier while streaming) and topk_stream_kernel (k <= 2048: a buffer cut by the whole CTA at a
// rendezvous).  Rows of at most 4096 elements are sorted whole in shared memory instead; rows
// split over several CTAs are merged by a second, tiny kernel.
#define TPB_FILE_ID 2
#include "common.cuh"
#include "host_util.h"

#include <algorithm>
#include <mutex>
#include <string>

namespace tpb {

constexpr int kMaxStreamWarps = 16;                            // a streaming CTA has 8 or 16 warps
constexpr int kWarpTile = 32 * 32;                            // 1024 elements per warp and iteration
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

// Compare-exchange steps of a bitonic network on 128 words held by one warp, four per lane
// (lane l holds positions pos0 + 4l .. pos0 + 4l + 3 of the whole array): the strides
// first_stride, first_stride/2, ..., 1 (first_stride <= 64) of the merge phase with block `size`.
// Strides below 4 stay inside a lane, the others are shuffles; no shared memory, no barrier.
__device__ __forceinline__ void warp_bitonic_steps(unsigned long long (&v)[4], int lane, int pos0, int size,
                                                   int first_stride) {
    for (int stride = first_stride; stride > 0; stride >>= 1) {
        if (stride < 4) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                if ((e & stride) == 0) {
                    const bool desc = (((pos0 + lane * 4 + e) & size) == 0);
                    const unsigned long long x = v[e], y = v[e | stride];
                    const bool sw = (x < y) == desc;
                    v[e] = sw ? y : x;
                    v[e | stride] = sw ? x : y;
                }
            }
        } else {
            const int ls = stride >> 2;
            const bool lower = (lane & ls) == 0;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const bool desc = (((pos0 + lane * 4 + e) & size) == 0);
                const unsigned long long o = __shfl_xor_sync(0xffffffffu, v[e], ls);
                const bool keep_max = lower == desc;
                const bool o_bigger = o > v[e];
                v[e] = (keep_max == o_bigger) ? o : v[e];
            }
        }
    }
}

// Descending bitonic sort of a[0..n), n a power of two, by all threads of the CTA (called by every
// thread).  For n >= 128 and whole warps, every run of strides below 128 is done by one warp per
// 128-word block in registers, so only the strides of 128 and more go through shared memory with a
// barrier each: 15 barriers instead of 66 for 2048 words.
__device__ void bitonic_desc(unsigned long long* a, int n, int tid, int nthr) {
    if (n >= 128 && (nthr & 31) == 0) {
        const int lane = tid & 31, warp = tid >> 5, nwarp = nthr >> 5;
        for (int blk = warp; blk < (n >> 7); blk += nwarp) {
            const int pos0 = blk << 7;
            unsigned long long v[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) v[e] = a[pos0 + lane * 4 + e];
            for (int size = 2; size <= 128; size <<= 1) warp_bitonic_steps(v, lane, pos0, size, size >> 1);
#pragma unroll
            for (int e = 0; e < 4; ++e) a[pos0 + lane * 4 + e] = v[e];
        }
        __syncthreads();
        for (int size = 256; size <= n; size <<= 1) {
            for (int stride = size >> 1; stride >= 128; stride >>= 1) {
                for (int t = tid; t < (n >> 1); t += nthr) {
                    const int lo = ((t & ~(stride - 1)) << 1) | (t & (stride - 1));
                    const int hi = lo | stride;
                    const bool desc = (lo & size) == 0;
                    const unsigned long long x = a[lo], y = a[hi];
                    if ((x < y) == desc) { a[lo] = y; a[hi] = x; }
                }
                __syncthreads();
            }
            for (int blk = warp; blk < (n >> 7); blk += nwarp) {
                const int pos0 = blk << 7;
                unsigned long long v[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) v[e] = a[pos0 + lane * 4 + e];
                warp_bitonic_steps(v, lane, pos0, size, 64);
#pragma unroll
                for (int e = 0; e < 4; ++e) a[pos0 + lane * 4 + e] = v[e];
            }
            __syncthreads();
        }
        return;
    }
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
    int warps;            // warps per streaming CTA (8 or 16)
};

__device__ __forceinline__ const float* topk_row(const float* in, const TopkGeom& g, long long r) {
    long long a = r / g.k1;
    long long b = r - a * g.k1;
    return in + a * g.ks0 + b * g.ks1;
}

// ------------------------------------------------------------------ streaming kernel -------
// Every warp streams its own tiles (warp w of NW takes warp-tiles w, w+NW, ... of the slice) with plain
// 128-bit streaming loads, eight per lane and iteration (1024 elements per warp-tile), exactly
// like the reduction kernels that reach the HBM roofline.  There is no CTA-wide barrier in the
// streaming loop; the warps of a CTA meet only at a "rendezvous" when the candidate buffer must be
// cut (a warp asks for it through a flag that every warp reads once per tile) and at the end.
// (A shared-memory ring filled by cp.async.bulk was measured first: with one 16 KB stage per CTA
// tile or one 2 KB stage per warp tile it kept too few bytes in flight per SM and spent its issue
// slots polling mbarriers: 71-125 us on the [256,151936] batch against 40 us for this form.)
struct StreamShared {
    unsigned long long tau;         // exclusive threshold: candidate iff word > tau (0 = none yet)
    unsigned long long samp[128];   // sorted sample of the buffer (cut)
    unsigned long long wmin[kMaxStreamWarps];  // per-warp bound of the bootstrap
    float tvf;                      // value of tau's key: the float prefilter compares against it
    int mode;                       // 0 accept everything, 1 float prefilter, 2 integer compare only
    int soft;                       // buffer fill at which a cut is requested
    int cnt;                        // words in the buffer (reservations may overshoot B)
    int request;                    // a warp asks every warp to the rendezvous
    int done;                       // warps that have streamed all their tiles
    int err;                        // a bounded wait gave up (give-up code)
    int arrive;                     // warps that have arrived at a rendezvous, over all rounds
    int tmp;
};

template <bool LARGEST>
__device__ __forceinline__ float worst_value() { return LARGEST ? -INFINITY : INFINITY; }

// Descending bitonic sort of 32*E words held by one warp, E per lane, lane-major ("blocked":
// lane l holds positions l*E .. l*E+E-1).  Strides below E are compare-exchanges inside a lane,
// the others are shuffles; no shared memory and no barrier.
template <int E, class T = unsigned long long>
__device__ __forceinline__ void warp_sort_desc(T (&v)[E], int lane) {
#pragma unroll
    for (int size = 2; size <= 32 * E; size <<= 1) {
#pragma unroll
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            if (stride < E) {
#pragma unroll
                for (int e = 0; e < E; ++e) {
                    if ((e & stride) == 0) {
                        const bool desc = (((lane * E + e) & size) == 0);
                        T x = v[e], y = v[e | stride];
                        const bool sw = (x < y) == desc;
                        v[e] = sw ? y : x;
                        v[e | stride] = sw ? x : y;
                    }
                }
            } else {
                const int ls = stride / E;
                const bool lower = (lane & ls) == 0;
#pragma unroll
                for (int e = 0; e < E; ++e) {
                    const bool desc = (((lane * E + e) & size) == 0);
                    T o = __shfl_xor_sync(kFull, v[e], ls);
                    const bool keep_max = lower == desc;
                    const bool o_bigger = o > v[e];
                    v[e] = (keep_max == o_bigger) ? o : v[e];
                }
            }
        }
    }
}

// Cut the candidate buffer back towards its k best and raise the threshold.  Entered by every
// thread after a barrier that made all appends visible.
//   n <= 256          warp 0 sorts the buffer in registers: exact, cnt = min(n, k)
//   n  > 256          sample-select: warp 0 sorts 128 evenly spaced samples, a sample is taken as
//                     pivot so that about 1.2 k words are expected at or above it, the words
//                     >= pivot are counted and -- if at least k and at most B/2 -- moved to the
//                     front (unordered).  O(n) work instead of a sort; the threshold becomes
//                     pivot - 1, a valid bound because at least k words lie above it.
//                     If three pivots fail, an exact CTA-wide bitonic sort is used instead.
//   final             the best min(n, k) are left SORTED in buf[0..), as the output needs them.
// Warp 0 sorts buf[0..n), n <= 256, descending in registers and writes it back padded with zeros
// to the next multiple of 32*E; the network size follows n (64, 128 or 256 words).
template <int E>
__device__ __forceinline__ void warp_sort_smem(unsigned long long* buf, int n, int lane) {
    unsigned long long v[E];
#pragma unroll
    for (int e = 0; e < E; ++e) v[e] = (lane * E + e) < n ? buf[lane * E + e] : 0ull;
    warp_sort_desc<E>(v, lane);
#pragma unroll
    for (int e = 0; e < E; ++e) buf[lane * E + e] = v[e];
}
__device__ __forceinline__ void warp_sort_upto256(unsigned long long* buf, int n, int lane) {
    if (n <= 64) warp_sort_smem<2>(buf, n, lane);
    else if (n <= 128) warp_sort_smem<4>(buf, n, lane);
    else warp_sort_smem<8>(buf, n, lane);
}

__device__ void cut(unsigned long long* buf, unsigned long long* buf2, StreamShared* sh, int B, int k,
                    int tid, int nthr, bool final) {
    const int lane = tid & 31;
    int n = sh->cnt;
    if (n > B) n = B;
    __syncthreads();   // everyone has read cnt before it is rewritten

    bool exact_needed = final;
    if (n > 256 && (!final || n > k + (k >> 1) + 64)) {
        if (tid < 32) {
            unsigned long long v[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) v[e] = buf[(long long)(tid * 4 + e) * n / 128];
            warp_sort_desc<4>(v, tid);
#pragma unroll
            for (int e = 0; e < 4; ++e) sh->samp[tid * 4 + e] = v[e];
        }
        __syncthreads();
        // sample rank whose pivot is expected to keep about 1.19 k + 24 words
        int q = (int)(((long long)128 * (k + (k >> 3) + (k >> 4) + 24) + n - 1) / n) + 1;
        bool ok = false;
        for (int attempt = 0; attempt < 3 && q <= 127; ++attempt, q += 8) {
            const unsigned long long pivot = sh->samp[q];
            if (tid == 0) sh->tmp = 0;
            __syncthreads();
            int c = 0;
            for (int i = tid; i < n; i += nthr) c += buf[i] >= pivot ? 1 : 0;
            c = __reduce_add_sync(kFull, c);
            if (lane == 0 && c) atomicAdd(&sh->tmp, c);
            __syncthreads();
            const int total = sh->tmp;
            __syncthreads();
            if (total >= k && total <= (B >> 1)) {
                if (tid == 0) sh->tmp = 0;
                __syncthreads();
                for (int base = 0; base < n; base += nthr) {
                    const int i = base + tid;
                    unsigned long long w = i < n ? buf[i] : 0ull;
                    const bool keep = w >= pivot;   // pivot > 0, so padding never passes
                    const unsigned bal = __ballot_sync(kFull, keep);
                    int wb = 0;
                    if (lane == 0 && bal) wb = atomicAdd(&sh->tmp, __popc(bal));
                    wb = __shfl_sync(kFull, wb, 0);
                    if (keep) buf2[wb + __popc(bal & ((1u << lane) - 1u))] = w;
                }
                __syncthreads();
                for (int i = tid; i < total; i += nthr) buf[i] = buf2[i];
                if (tid == 0) { sh->cnt = total; sh->tau = pivot - 1ull; }
                __syncthreads();
                n = total;
                ok = true;
                break;
            }
        }
        if (!ok) exact_needed = true;
    } else {
        exact_needed = true;
    }
    if (!exact_needed) return;

    if (n <= 256) {
        if (tid < 32) {
            warp_sort_upto256(buf, n, tid);
            __syncwarp();
            if (tid == 0) {
                sh->cnt = n < k ? n : k;
                sh->tau = n >= k ? buf[k - 1] : 0ull;
            }
        }
        __syncthreads();
        return;
    }
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

// What the rendezvous decided (identical in every thread).
enum { kActCut = 0, kActFinal = 1 };
// Give-up codes left in the status word (low byte; the rendezvous round follows in the next bits).
enum { kErrRendezvous = 2, kErrRetry = 3, kErrPolling = 4 };

// The body of the rendezvous kernel: slice s of row r (row points at the row's first element), with
// the candidate buffer buf (g.B words), the partition target buf2 (g.B / 2 words) and the control
// block sh in the caller's shared memory.  Called by every thread of a CTA of NW warps.  It is the
// whole of topk_stream_kernel, and topk_select_kernel calls it on the rows that fail its check.
template <bool LARGEST, bool VEC, int NW>
__device__ __forceinline__ void stream_body(const float* __restrict__ row, const TopkGeom& g, int s, long long r,
                                            unsigned long long* buf, unsigned long long* buf2, StreamShared& sh,
                                            unsigned long long* __restrict__ ws, float* __restrict__ out_val,
                                            long long* __restrict__ out_idx, int* status) {
    constexpr int kStreamWarps = NW;
    constexpr int kStreamThreads = NW * 32;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const long long begin = (long long)s * g.chunk;
    long long len = g.len - begin;
    if (len > g.chunk) len = g.chunk;
    const float* slice = row + begin * g.es;
    const int ntiles = (int)((len + kWarpTile - 1) / kWarpTile);       // warp-tiles in the slice
    const int my_tiles = ntiles > warp ? (ntiles - warp + kStreamWarps - 1) / kStreamWarps : 0;
    const int B = g.B, k = (int)g.k;

    if (tid == 0) {
        sh.tau = 0ull; sh.tvf = worst_value<LARGEST>(); sh.mode = 0; sh.soft = g.soft;
        sh.cnt = 0; sh.request = 0; sh.done = 0; sh.err = 0; sh.arrive = 0; sh.tmp = 0;
    }
    __syncthreads();

    // Rendezvous of the CTA's warps (no warp is appending while it lasts).  The hardware barrier is
    // entered only after a software arrival count shows that all of them are present: a warp
    // that never comes therefore cannot hang the others -- the wait is bounded, gives up with an
    // error code in the status word, and everybody leaves.  Cuts the buffer, or, once all warps have
    // finished streaming (or after a failure), says so -- the same answer in every thread.
    int round = 0;
    auto give_up = [&](int code) {
        if (lane == 0) {
            *(volatile int*)&sh.err = code;
            *(volatile int*)&sh.request = 1;
            if (status) atomicMax(status, code | (round << 8));
        }
    };
    auto rendezvous = [&]() -> int {
        __syncwarp();
        ++round;
        if (lane == 0) atomicAdd(&sh.arrive, 1);
        const int target = round * kStreamWarps;
        bool here = false;
        for (int spin = 0; spin < (1 << 21); ++spin) {
            if (*(volatile int*)&sh.arrive >= target || *(volatile int*)&sh.err) { here = true; break; }
            __nanosleep(40);
        }
        here = __all_sync(kFull, here);
        if (!here) give_up(kErrRendezvous);
        if (!here || *(volatile int*)&sh.err) return kActFinal;   // nobody touches the barrier after a failure
        __syncthreads();
        const bool fin = *(volatile int*)&sh.done == kStreamWarps;
        if (fin) return kActFinal;
        cut(buf, buf2, &sh, B, k, tid, kStreamThreads, false);
        if (tid == 0) {
            const unsigned long long t = sh.tau;
            sh.mode = t == 0ull ? 0 : ((t >> 32) == 0ull ? 2 : 1);
            sh.tvf = key_value<LARGEST>((unsigned)(t >> 32));
            sh.soft = B;            // after the first cut only a full buffer asks for another
            sh.request = 0;
        }
        __syncthreads();
        return kActCut;
    };

    // Element j (0..31) of this lane in the warp's tile at offset `off` of the slice is element
    // ((j>>2)*32 + lane)*4 + (j&3) of the tile: float4 number u*32+lane, component c, j = 4u+c.
    auto elem_off = [&](long long off, int j) -> long long { return off + ((j >> 2) * 32 + lane) * 4 + (j & 3); };

    // ---- bootstrap (k <= 8 per warp, slice of at least one tile per warp): each warp sorts the 32
    // per-lane maxima of its first tile with shuffles; with j = ceil(k / warps) every warp holds j
    // lane maxima at or above its j-th largest, so the smallest of the warps' j-th largest values
    // has at least warps * j >= k elements at or above it: a valid starting threshold.
    const bool boot = k <= 8 * kStreamWarps && len >= (long long)kStreamWarps * kWarpTile;
    if (boot) {
        const long long off = (long long)warp * kWarpTile;
        unsigned long long gm[1] = {0ull};
        if (VEC) {
            const float* p = slice + off + lane * 4;
            float4 v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) v[u] = ld_keep4(p + u * 128);
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const unsigned b0 = (unsigned)(begin + off) + (u * 32 + lane) * 4;
                unsigned long long w;
                w = rank_word<LARGEST>(v[u].x, b0);     gm[0] = w > gm[0] ? w : gm[0];
                w = rank_word<LARGEST>(v[u].y, b0 + 1); gm[0] = w > gm[0] ? w : gm[0];
                w = rank_word<LARGEST>(v[u].z, b0 + 2); gm[0] = w > gm[0] ? w : gm[0];
                w = rank_word<LARGEST>(v[u].w, b0 + 3); gm[0] = w > gm[0] ? w : gm[0];
            }
        } else {
#pragma unroll 8
            for (int j = 0; j < 32; ++j) {
                const long long e = elem_off(off, j);
                unsigned long long w = rank_word<LARGEST>(ld_stream1(slice + e * g.es), (unsigned)(begin + e));
                gm[0] = w > gm[0] ? w : gm[0];
            }
        }
        warp_sort_desc<1>(gm, lane);
        const unsigned long long jth = __shfl_sync(kFull, gm[0], (k + kStreamWarps - 1) / kStreamWarps - 1);
        if (lane == 0) sh.wmin[warp] = jth;
        __syncthreads();
        if (tid == 0) {
            unsigned long long t = sh.wmin[0];
            for (int w8 = 1; w8 < kStreamWarps; ++w8) t = sh.wmin[w8] < t ? sh.wmin[w8] : t;
            t -= 1ull;   // exclusive; the low word of a rank word is never 0, so no borrow from the key
            sh.tau = t;
            sh.mode = (t >> 32) == 0ull ? 2 : 1;
            sh.tvf = key_value<LARGEST>((unsigned)(t >> 32));
        }
        __syncthreads();
    } else if (k <= 128 * kStreamWarps && len >= (long long)kStreamWarps * kWarpTile) {
        // ---- bootstrap for 8 < k / warps <= 128: the same bound from FOUR values per lane (a
        // tighter one than the lane maxima give once j approaches 32: measured on [512, 2^20],
        // k = 512: 432 -> 415 us).  Every
        // lane keeps the four best of its 32 elements as plain floats (a min/max insertion chain,
        // NaN ignored), the warp sorts the 128 as keys and offers its j-th largest, j = ceil(k /
        // warps); the smallest offer has at least warps * j >= k elements at or above its value.  A
        // lane with fewer than four numbers leaves its start value in the list; if an offer is that
        // start value the row gets no threshold here and begins by taking everything, as it would
        // without a bootstrap.  (On [512, 2^20], k = 1024, starting without a threshold costs two of
        // five cuts and a third of the candidates.)
        const long long off = (long long)warp * kWarpTile;
        const float worst = worst_value<LARGEST>();
        float f0 = worst, f1 = worst, f2 = worst, f3 = worst;
        auto take = [&](float a) {
            float hi;
            hi = LARGEST ? fmaxf(f0, a) : fminf(f0, a); a = LARGEST ? fminf(f0, a) : fmaxf(f0, a); f0 = hi;
            hi = LARGEST ? fmaxf(f1, a) : fminf(f1, a); a = LARGEST ? fminf(f1, a) : fmaxf(f1, a); f1 = hi;
            hi = LARGEST ? fmaxf(f2, a) : fminf(f2, a); a = LARGEST ? fminf(f2, a) : fmaxf(f2, a); f2 = hi;
            f3 = LARGEST ? fmaxf(f3, a) : fminf(f3, a);
        };
        if (VEC) {
            const float* p = slice + off + lane * 4;
            float4 v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) v[u] = ld_keep4(p + u * 128);
#pragma unroll
            for (int u = 0; u < 8; ++u) { take(v[u].x); take(v[u].y); take(v[u].z); take(v[u].w); }
        } else {
#pragma unroll 8
            for (int j = 0; j < 32; ++j) take(ld_stream1(slice + elem_off(off, j) * g.es));
        }
        unsigned kk[4] = {rank_key<LARGEST>(f0), rank_key<LARGEST>(f1), rank_key<LARGEST>(f2), rank_key<LARGEST>(f3)};
        warp_sort_desc<4, unsigned>(kk, lane);
        const int jr = (k + kStreamWarps - 1) / kStreamWarps - 1;     // 0-based rank among the warp's 128 keys
        unsigned sel = kk[0];
#pragma unroll
        for (int e = 1; e < 4; ++e) sel = (jr & 3) == e ? kk[e] : sel;
        sel = __shfl_sync(kFull, sel, jr >> 2);
        if (lane == 0) sh.wmin[warp] = (unsigned long long)sel;
        __syncthreads();
        if (tid == 0) {
            unsigned lo = (unsigned)sh.wmin[0];
            for (int w8 = 1; w8 < kStreamWarps; ++w8) lo = (unsigned)sh.wmin[w8] < lo ? (unsigned)sh.wmin[w8] : lo;
            if (lo > rank_key<LARGEST>(worst)) {
                // exclusive threshold below every element of that key: the low half of a word is never 0
                const unsigned long long t = (unsigned long long)lo << 32;
                sh.tau = t;
                sh.mode = 1;
                sh.tvf = key_value<LARGEST>(lo);
            }
        }
        __syncthreads();
    }

    // ---- streaming loop (warp-autonomous)
    // Hot path: eight 128-bit loads per lane, 32 float compares, one 32-bit mask; nothing else is
    // kept.  The loads allocate in L1 (ld_keep4): with k in the hundreds a tile holds ten or more
    // candidates, and on inputs far larger than L2 their re-reads went to DRAM when the tile was
    // loaded past L1 (ncu on [512, 2^20], k = 1024: 6.6 % more DRAM bytes than the input; 477 us
    // with streaming loads, 439 us with these).  A set bit is a possible candidate: its element is read again by address (an L2 hit),
    // ranked exactly on the 64-bit word, and appended with one shared-memory atomic.
    // `abort`: a rendezvous reported a failure somewhere in the CTA; every warp saw the same answer
    // at the same rendezvous and leaves.
    bool abort = false;
    for (int i = 0; i < my_tiles && !abort; ++i) {
        const long long off = (long long)(warp + i * kStreamWarps) * kWarpTile;
        const int mode = __shfl_sync(kFull, *(volatile int*)&sh.mode, 0);
        unsigned m = 0u;
        if (mode == 1) {
            // prefilter: warps run at different places of the row, so an element that ties the
            // threshold value may still outrank it (lower index): keep ties, decide exactly below
            const float tvf = *(volatile float*)&sh.tvf;
            if (VEC && off + kWarpTile <= len) {
                const float* p = slice + off + lane * 4;
                float4 v[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) v[u] = ld_keep4(p + u * 128);
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const bool p0 = LARGEST ? (v[u].x >= tvf) : (v[u].x <= tvf);
                    const bool p1 = LARGEST ? (v[u].y >= tvf) : (v[u].y <= tvf);
                    const bool p2 = LARGEST ? (v[u].z >= tvf) : (v[u].z <= tvf);
                    const bool p3 = LARGEST ? (v[u].w >= tvf) : (v[u].w <= tvf);
                    m |= (p0 ? 1u : 0u) << (4 * u) | (p1 ? 2u : 0u) << (4 * u) | (p2 ? 4u : 0u) << (4 * u) |
                         (p3 ? 8u : 0u) << (4 * u);
                }
            } else {
#pragma unroll 8
                for (int j = 0; j < 32; ++j) {
                    const long long e = elem_off(off, j);
                    if (e < len) {
                        const float xv = ld_stream1(slice + e * g.es);
                        const bool pj = LARGEST ? (xv >= tvf) : (xv <= tvf);
                        m |= pj ? (1u << j) : 0u;
                    }
                }
            }
        } else {
            m = 0xffffffffu;   // no usable float threshold yet: every element is ranked exactly
        }
        int retries = 0;
        while (__any_sync(kFull, m != 0u)) {
            if (++retries > 4096) { give_up(kErrRetry); abort = true; break; }   // a cut always frees slots
            const unsigned long long tau = *(volatile unsigned long long*)&sh.tau;
            bool over = false;
            while (m != 0u) {
                const int j = __ffs(m) - 1;
                const long long e = elem_off(off, j);
                if (e < len) {
                    const float xv = *TPB_CK(&slice[e * g.es]);
                    const unsigned long long w = rank_word<LARGEST>(xv, (unsigned)(begin + e));
                    if (w > tau) {
                        const int pos = atomicAdd(&sh.cnt, 1);
                        if (pos >= B) { over = true; break; }    // keep the bit: retried after the cut
                        buf[pos] = w;
                        if (pos + 1 > *(volatile int*)&sh.soft) *(volatile int*)&sh.request = 1;
                    }
                }
                m &= m - 1u;
            }
            __syncwarp();
            if (!__any_sync(kFull, over)) break;
            // the buffer is full: meet the other warps, cut, and retry what still qualifies
            if (lane == 0) *(volatile int*)&sh.request = 1;
            __syncwarp();
            if (rendezvous() == kActFinal) { abort = true; break; }
        }
        // one lane reads the flag for the whole warp: the decision to meet must be warp-uniform
        __syncwarp();
        const int req = __shfl_sync(kFull, *(volatile int*)&sh.request | *(volatile int*)&sh.err, 0);
        if (!abort && req) {
            if (rendezvous() == kActFinal) abort = true;
        }
    }

    // ---- this warp has no tiles left: keep answering rendezvous requests until all warps are done.
    // The polling is bounded (about 0.3 s): on give-up the failure is recorded and the kernel ends.
    if (!abort) {
        __syncwarp();
        if (lane == 0) atomicAdd(&sh.done, 1);
        __syncwarp();
        for (int spin = 0;; ++spin) {
            int go = (*(volatile int*)&sh.request != 0) | (*(volatile int*)&sh.done == kStreamWarps) |
                     (*(volatile int*)&sh.err != 0);
            go = __shfl_sync(kFull, go, 0);
            if (go) {
                if (rendezvous() == kActFinal) break;
                spin = 0;
            } else {
                if (spin > (1 << 21)) { give_up(kErrPolling); break; }
                __nanosleep(40);
            }
        }
    }
    if (*(volatile int*)&sh.err) {
        if (tid == 0 && status) atomicMax(status, 1);
        return;   // outputs stay unwritten; the host reads the status word
    }

    // ---- final cut: the slice's best min(cnt, k), sorted
    cut(buf, buf2, &sh, B, k, tid, kStreamThreads, true);
    const int cnt = sh.cnt;
    if (ws) {
        unsigned long long* dst = ws + ((size_t)r * g.S + s) * (size_t)k;
        for (int j = tid; j < k; j += kStreamThreads) *TPB_CK(&dst[j]) = j < cnt ? buf[j] : 0ull;
    } else {
        for (int j = tid; j < k && j < cnt; j += kStreamThreads) {
            const unsigned long long w = buf[j];
            const unsigned idx = word_index(w);
            const unsigned key = (unsigned)(w >> 32);
            float val = key_value<LARGEST>(key);
            // the key folds -0.0 onto +0.0 and all NaNs onto one rank: those come from the row
            if (key == 0u || val == 0.0f) val = *TPB_CK(&row[(long long)idx * g.es]);
            *TPB_CK(&out_idx[r * k + j]) = (long long)idx;
            *TPB_CK(&out_val[r * k + j]) = val;
        }
    }
}

// The same as a real function, for topk_select_kernel: the geometry travels by value, so the body
// works on a private copy that no store can alias.
template <bool LARGEST, bool VEC, int NW>
__device__ __noinline__ void stream_body_call(const float* __restrict__ row, TopkGeom g, long long r,
                                              unsigned long long* buf, StreamShared& sh, float* __restrict__ out_val,
                                              long long* __restrict__ out_idx, int* status) {
    stream_body<LARGEST, VEC, NW>(row, g, 0, r, buf, buf + g.B, sh, nullptr, out_val, out_idx, status);
}

template <bool LARGEST, bool VEC, int NW>
__global__ void __launch_bounds__(NW * 32, 32 / NW)
topk_stream_kernel(const float* __restrict__ in, TopkGeom g, unsigned long long* __restrict__ ws,
                   float* __restrict__ out_val, long long* __restrict__ out_idx, int* status) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    unsigned long long* buf = reinterpret_cast<unsigned long long*>(smem_raw);
    __shared__ StreamShared sh;
    const int s = (int)(blockIdx.x % (unsigned)g.S);
    const long long r = (long long)(blockIdx.x / (unsigned)g.S);
    stream_body<LARGEST, VEC, NW>(topk_row(in, g, r), g, s, r, buf, buf + g.B, sh, ws, out_val, out_idx, status);
}

// ------------------------------------------------------------------ small-k streaming kernel
// k <= 64.  Same one-pass idea as topk_stream_kernel, but after the bootstrap NO barrier of the CTA
// is left, candidates never go back to memory, and a cut never stops the other warps:
//  * the warps take 1024-element tiles from a shared counter;
//  * the threshold test is one float compare per element and leaves a 32-bit mask per lane; the few
//    elements that pass are read again by address (an L2 hit), ranked exactly (64-bit word) and
//    appended, one shared-memory atomic each, to a RING of 1024 words whose write position only grows;
//  * the ring is consumed in chunks of 64 words.  The warp whose reservation completes chunk c cuts
//    it: it waits (bounded) for chunk c-1 to be done and for the 64 slots to be written (an empty
//    slot is 0, a rank word never is), sorts them together with the 64 survivors of the earlier
//    chunks in registers (128 words, four per lane, about a microsecond), leaves the best 64 as
//    the new survivors, raises the threshold to the k-th of them, zeroes the slots and advances
//    `consumed`.  Meanwhile the other warps stream on; they only wait if the ring is full, i.e. if
//    the cuts are 15 chunks behind;
//  * the warp that leaves last merges the unfinished chunk with the survivors and writes the output.
// A lane whose reservation completes a chunk, or finds the ring full, stops appending; the warp
// then handles these events in ascending ring position (write the word once there is room, cut the
// chunk) before any lane reserves again.  Waits therefore only ever depend on lower positions and
// cannot form a cycle; every wait is bounded all the same and ends with a code in the status word
// and unwritten outputs.
constexpr int kSmallK = 64;
constexpr int kRing = 1024;
constexpr int kChunk = 64;
constexpr int kSmallSpin = 1 << 22;
enum { kErrSlot = 6, kErrRingFull = 7, kErrChunkOrder = 8 };

struct SmallShared {
    unsigned long long tau;        // exclusive threshold, only ever raised
    unsigned long long best[64];   // survivors of the chunks cut so far, sorted descending, 0-padded
    unsigned bootk[128];           // bootstrap: the warps' largest lane maxima (as keys)
    unsigned cnt;                  // words ever reserved in the ring
    unsigned consumed;             // words taken over by cuts
    int next;                      // next warp-tile of the slice
    int done;                      // warps that have left the streaming loop
    int err;
};

// Bounded wait for a ring slot to be written; 0 on give-up.
__device__ __forceinline__ unsigned long long wait_slot(const unsigned long long* p, const int* err) {
    unsigned long long w = *(const volatile unsigned long long*)p;
    for (int spin = 0; w == 0ull && spin < kSmallSpin; ++spin) {
        if (*(const volatile int*)err) break;
        __nanosleep(20);
        w = *(const volatile unsigned long long*)p;
    }
    return w;
}

__device__ __forceinline__ void small_give_up(SmallShared* sh, int* status, int code, int lane) {
    if (lane == 0) {
        *(volatile int*)&sh->err = code;
        if (status) atomicMax(status, code);
    }
}

// Warp-uniform bounded wait until `consumed` has reached `target`; false on give-up.
__device__ __noinline__ bool wait_consumed(SmallShared* sh, unsigned target, int lane) {
    int ok = 0;
    if (lane == 0) {
        for (int spin = 0; spin < kSmallSpin; ++spin) {
            if (*(volatile unsigned*)&sh->consumed >= target) { ok = 1; break; }
            if (*(volatile int*)&sh->err) break;
            __nanosleep(40);
        }
    }
    return __shfl_sync(kFull, ok, 0) != 0;
}

// Cut chunk c of the ring (called by one whole warp).  n_new = words of the chunk (kChunk, or
// fewer for the unfinished chunk at the end).  Leaves the sorted union's best 64 in sh->best;
// false on give-up.
__device__ __noinline__ bool cut_chunk(unsigned long long* ring, SmallShared* sh, unsigned c, int n_new, int k,
                                       int lane, int* status) {
    unsigned long long v[4];
    if (!wait_consumed(sh, c * kChunk, lane)) { small_give_up(sh, status, kErrChunkOrder, lane); return false; }
    bool ok = true;
#pragma unroll
    for (int e = 0; e < 2; ++e) {
        const int i = lane * 2 + e;
        v[e] = 0ull;
        if (i < n_new) {
            unsigned long long* slot = &ring[(c * kChunk + i) & (kRing - 1)];
            v[e] = wait_slot(slot, &sh->err);
            ok &= v[e] != 0ull;
            *(volatile unsigned long long*)slot = 0ull;
        }
    }
    v[2] = sh->best[lane * 2];
    v[3] = sh->best[lane * 2 + 1];
    if (!__all_sync(kFull, ok)) { small_give_up(sh, status, kErrSlot, lane); return false; }
    warp_sort_desc<4>(v, lane);
    if (lane < 16) {
#pragma unroll
        for (int e = 0; e < 4; ++e) sh->best[lane * 4 + e] = v[e];
    }
    unsigned long long sel = v[0];
#pragma unroll
    for (int e = 1; e < 4; ++e) sel = ((k - 1) & 3) == e ? v[e] : sel;
    const unsigned long long kth = __shfl_sync(kFull, sel, (k - 1) >> 2);
    __syncwarp();
    if (lane == 0) {
        // fewer than k words so far (kth == 0) leaves the threshold alone
        if (kth != 0ull && kth - 1ull > *(volatile unsigned long long*)&sh->tau) *(volatile unsigned long long*)&sh->tau = kth - 1ull;
        __threadfence_block();
        *(volatile unsigned*)&sh->consumed = c * kChunk + n_new;
    }
    __syncwarp();
    return true;
}

template <bool LARGEST, bool VEC, int NW>
__global__ void __launch_bounds__(NW * 32, NW == 4 ? 7 : (NW == 8 ? 4 : 2))
topk_smallk_kernel(const float* __restrict__ in, TopkGeom g, unsigned long long* __restrict__ ws,
                   float* __restrict__ out_val, long long* __restrict__ out_idx, int* status) {
    __shared__ __align__(16) unsigned long long ring[kRing];
    __shared__ SmallShared sh;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int s = (int)(blockIdx.x % (unsigned)g.S);
    const long long r = (long long)(blockIdx.x / (unsigned)g.S);
    const float* row = topk_row(in, g, r);
    const long long begin = (long long)s * g.chunk;
    long long len = g.len - begin;
    if (len > g.chunk) len = g.chunk;
    const float* slice = row + begin * g.es;
    const int ntiles = (int)((len + kWarpTile - 1) / kWarpTile);
    const int k = (int)g.k;

    for (int i = tid; i < kRing; i += NW * 32) ring[i] = 0ull;
    if (tid < 64) sh.best[tid] = 0ull;
    if (tid == 0) { sh.tau = 0ull; sh.cnt = 0u; sh.consumed = 0u; sh.next = 2 * NW; sh.done = 0; sh.err = 0; }   // tiles 0 .. 2 NW - 1 are taken by the bootstrap

    // Element j (0..31) of this lane in the tile at offset `off`: float4 number u*32+lane, component
    // c, j = 4u+c.
    auto elem_off = [&](long long off, int j) -> long long { return off + ((j >> 2) * 32 + lane) * 4 + (j & 3); };

    // A tile in registers.  Elements past the end of the slice read as NaN.
    auto load_tile = [&](float4 (&v)[8], long long off) {
        if (VEC && off + kWarpTile <= len) {
            const float* p = slice + off + lane * 4;
#pragma unroll
            for (int u = 0; u < 8; ++u) v[u] = ld_stream4(p + u * 128);
        } else {
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const long long e0 = off + (u * 32 + lane) * 4;
                float t[4];
#pragma unroll
                for (int c = 0; c < 4; ++c) t[c] = e0 + c < len ? ld_stream1(slice + (e0 + c) * g.es) : NAN;
                v[u] = make_float4(t[0], t[1], t[2], t[3]);
            }
        }
    };

    // Bit j set: element j of this lane may beat the threshold.  The float test lets ties with the
    // threshold value pass (a tie with a lower index outranks it); the exact compare decides later.
    auto mask_of = [&](const float4 (&v)[8], unsigned long long tau) -> unsigned {
        if ((tau >> 32) == 0ull) return 0xffffffffu;   // the threshold's key is 0 (NaN rank): rank everything
        const float tvf = key_value<LARGEST>((unsigned)(tau >> 32));
        unsigned m = 0u;
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const bool p0 = LARGEST ? (v[u].x >= tvf) : (v[u].x <= tvf);
            const bool p1 = LARGEST ? (v[u].y >= tvf) : (v[u].y <= tvf);
            const bool p2 = LARGEST ? (v[u].z >= tvf) : (v[u].z <= tvf);
            const bool p3 = LARGEST ? (v[u].w >= tvf) : (v[u].w <= tvf);
            m |= (p0 ? 1u : 0u) << (4 * u) | (p1 ? 2u : 0u) << (4 * u) | (p2 ? 4u : 0u) << (4 * u) |
                 (p3 ? 8u : 0u) << (4 * u);
        }
        return m;
    };

    // Append the masked elements of the tile at `off`; false after a give-up.
    auto drain = [&](unsigned m, long long off) -> bool {
        for (int pass = 0; __any_sync(kFull, m != 0u); ++pass) {
            if (pass > (1 << 22)) { small_give_up(&sh, status, kErrRetry, lane); return false; }
            const unsigned long long tnow = *(volatile unsigned long long*)&sh.tau;
            unsigned ev_pos = 0xffffffffu;     // a reservation of this lane that the warp must attend to
            unsigned long long ev_w = 0ull;
            int ev_kind = 0;                   // 1: not written yet, the ring was full;  2: completes a chunk
            while (m != 0u) {
                const int j = __ffs(m) - 1;
                m &= m - 1u;
                const long long e = elem_off(off, j);
                if (e < len) {
                    const float xv = *TPB_CK(&slice[e * g.es]);
                    const unsigned long long w = rank_word<LARGEST>(xv, (unsigned)(begin + e));
                    if (w > tnow) {
                        const unsigned pos = atomicAdd(&sh.cnt, 1u);
                        const bool full = pos - *(volatile unsigned*)&sh.consumed >= (unsigned)kRing;
                        if (!full) *(volatile unsigned long long*)&ring[pos & (kRing - 1)] = w;
                        const bool duty = (pos + 1u) % (unsigned)kChunk == 0u;
                        if (full || duty) {
                            ev_pos = pos; ev_w = w; ev_kind = (full ? 1 : 0) | (duty ? 2 : 0);
                            break;
                        }
                    }
                }
            }
            __syncwarp();
            for (;;) {   // events of the warp in ascending ring position (rare)
                const unsigned pmin = __reduce_min_sync(kFull, ev_pos);
                if (pmin == 0xffffffffu) break;
                const bool mine = ev_pos == pmin;
                const int src = __ffs(__ballot_sync(kFull, mine)) - 1;
                const int kind = __shfl_sync(kFull, ev_kind, src);
                if (kind & 1) {
                    if (!wait_consumed(&sh, pmin - (unsigned)kRing + 1u, lane)) { small_give_up(&sh, status, kErrRingFull, lane); return false; }
                    if (mine) *(volatile unsigned long long*)&ring[pmin & (kRing - 1)] = ev_w;
                    __syncwarp();
                }
                if (kind & 2) {
                    if (!cut_chunk(ring, &sh, pmin / (unsigned)kChunk, kChunk, k, lane, status)) return false;
                }
                if (mine) ev_pos = 0xffffffffu;
            }
        }
        return true;
    };

    // ---- bootstrap: warp w loads tile w and sorts its 32 lane maxima (as keys) with shuffles; the
    // 128/NW largest of every warp are put together and the k-th largest of those 128 -- found by
    // rank counting, one thread per key -- is the first threshold.  All 128 are distinct elements of
    // the row, so at least k elements reach it; it is almost always within a few ranks of the
    // exact k-th largest of the first NW*1024 elements.  (The planner guarantees len >= NW tiles.)
    bool failed = false;
    {
        float4 v[8];
        const long long off = (long long)warp * kWarpTile;
        if (VEC && off + kWarpTile <= len) {
            // with allocation in L1: the tile is read again below, once the threshold is known
            const float* p = slice + off + lane * 4;
#pragma unroll
            for (int u = 0; u < 8; ++u) v[u] = ld_keep4(p + u * 128);
        } else {
            load_tile(v, off);
        }
        float mx = NAN;   // fmaxf/fminf ignore a NaN operand: stays NaN only if the lane saw nothing else
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            if (LARGEST) mx = fmaxf(fmaxf(mx, v[u].x), fmaxf(fmaxf(v[u].y, v[u].z), v[u].w));
            else         mx = fminf(fminf(mx, v[u].x), fminf(fminf(v[u].y, v[u].z), v[u].w));
        }
        unsigned key = rank_key<LARGEST>(mx);
        // The lane maxima are all the bootstrap needs of its tile: the registers take the warp's first
        // streaming tile now, so that its loads are in flight while the threshold is worked out (the
        // sort, two barriers and the rank count below were 2 us in which this CTA loaded nothing).
        const long long off1 = (long long)(NW + warp) * kWarpTile;
        const bool has1 = NW + warp < ntiles;
        if (has1) load_tile(v, off1);
#pragma unroll
        for (int size = 2; size <= 32; size <<= 1) {
#pragma unroll
            for (int stride = size >> 1; stride > 0; stride >>= 1) {
                const unsigned o = __shfl_xor_sync(kFull, key, stride);
                const bool keep_max = ((lane & stride) == 0) == ((lane & size) == 0);
                key = keep_max ? (o > key ? o : key) : (o < key ? o : key);
            }
        }
        constexpr int kShare = 128 / NW;
        if (lane < kShare) sh.bootk[warp * kShare + lane] = key;
        __syncthreads();
        if (tid < 128) {
            const unsigned my = sh.bootk[tid];
            int above = 0, equal = 0;
            for (int i = 0; i < 128; ++i) {
                const unsigned o = sh.bootk[i];
                above += o > my ? 1 : 0;
                equal += o == my ? 1 : 0;
            }
            if (above < k && k <= above + equal) sh.tau = (unsigned long long)my << 32;   // same value from every writer
        }
        __syncthreads();
        const unsigned long long tau0 = *(volatile unsigned long long*)&sh.tau;
        if (has1) {
            const unsigned m1 = mask_of(v, tau0);
            if (!drain(m1, off1)) failed = true;
        }
        if (!failed) {
            load_tile(v, off);   // the bootstrap tile again (L1 / L2)
            const unsigned m = mask_of(v, *(volatile unsigned long long*)&sh.tau);
            if (!drain(m, off)) failed = true;
        }
    }

    // ---- streaming loop: no barrier, tiles from a shared counter
    while (!failed) {
        int t = 0;
        unsigned long long tau = 0ull;
        if (lane == 0) {
            t = atomicAdd(&sh.next, 1);
            tau = *(volatile unsigned long long*)&sh.tau;
            if (*(volatile int*)&sh.err) t = ntiles;
        }
        t = __shfl_sync(kFull, t, 0);
        tau = __shfl_sync(kFull, tau, 0);
        if (t >= ntiles) break;
        const long long off = (long long)t * kWarpTile;
        unsigned m;
        {
            float4 v[8];
            load_tile(v, off);
            m = mask_of(v, tau);
        }
        if (!drain(m, off)) failed = true;
    }

    // ---- the warp that leaves last merges the unfinished chunk with the survivors and writes the output
    __syncwarp();
    int last = 0;
    if (lane == 0) {
        __threadfence_block();
        last = atomicAdd(&sh.done, 1) == NW - 1;
    }
    last = __shfl_sync(kFull, last, 0);
    if (!last) return;
    if (*(volatile int*)&sh.err) {
        if (lane == 0 && status) atomicMax(status, 1);
        return;   // outputs stay unwritten; the host reads the status word
    }
    const unsigned total = *(volatile unsigned*)&sh.cnt;
    const unsigned c_last = total / (unsigned)kChunk;    // every complete chunk has been cut by its warp
    const int n_new = (int)(total - c_last * (unsigned)kChunk);
    if (!wait_consumed(&sh, c_last * (unsigned)kChunk, lane)) {
        small_give_up(&sh, status, kErrChunkOrder, lane);
        return;
    }
    auto emit = [&](unsigned long long w, int rank) {
        if (w == 0ull || rank >= k) return;
        if (ws) {
            *TPB_CK(&ws[((size_t)r * g.S + s) * (size_t)k + rank]) = w;
        } else {
            const unsigned idx = word_index(w);
            const unsigned key = (unsigned)(w >> 32);
            float val = key_value<LARGEST>(key);
            // the key folds -0.0 onto +0.0 and all NaNs onto one rank: those come from the row
            if (key == 0u || val == 0.0f) val = *TPB_CK(&row[(long long)idx * g.es]);
            *TPB_CK(&out_idx[r * k + rank]) = (long long)idx;
            *TPB_CK(&out_val[r * k + rank]) = val;
        }
    };
    if (!cut_chunk(ring, &sh, c_last, n_new, k, lane, status)) {
        if (lane == 0 && status) atomicMax(status, 1);
        return;
    }
    __syncwarp();
    emit(sh.best[lane * 2], lane * 2);
    emit(sh.best[lane * 2 + 1], lane * 2 + 1);
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
        for (int i = tid; i < N; i += nthr) buf[i] = i < n_items ? *TPB_CK(&src[i]) : 0ull;
    }
    __syncthreads();
    bitonic_desc(buf, N, tid, nthr);
    const int k = (int)g.k;
    for (int j = tid; j < k; j += nthr) {
        unsigned idx = word_index(buf[j]);
        // a slice kernel that gave up (status word set) leaves its words unwritten: never follow
        // an index that is not inside the row
        const bool inside = (long long)idx < g.len;
        *TPB_CK(&out_idx[r * k + j]) = inside ? (long long)idx : -1LL;
        *TPB_CK(&out_val[r * k + j]) = inside ? *TPB_CK(&row[(long long)idx * g.es]) : NAN;
    }
}

// ------------------------------------------------------------------ short rows, small k ----
// Rows of at most 4096 elements with k <= 64: one WARP per row (four rows per CTA), no barrier.
//   1. every lane keeps the keys of its two best elements while the row is loaded (all 32 x 2 are
//      distinct elements of the row); the k-th best of those 64 keys -- rank counting, two keys per
//      lane -- is a threshold that at least k elements reach (key 0 = "take everything" when the row
//      has fewer than k such keys);
//   2. the row is walked again (registers for one tile, L1 / L2 otherwise) and the elements that reach
//      the threshold are appended to the warp's 256-word buffer: per tile one mask per lane and one
//      prefix sum over the lanes' counts;
//   3. the buffer is sorted by the warp (bitonic network in shared memory) and the first k words are
//      written out.
// A row with more than 256 elements at or above its threshold (long runs of equal values) is done by
// selection instead: k times the best word below the last one, the row read from L1 each time --
// slow, exact, and only ever taken by such rows.
// (Sorting every such row whole in shared memory, one CTA per row, ran [65536,1024] k = 10 in
// 1454 us and [16384,4096] k = 50 in 1736 us: 3 % of the copy bandwidth.)
// The same idea for thousands of rows of 4 K to 64 K elements -- a warp per row in ONE pass, threshold
// from the first tile and raised by cuts of the warp's buffer -- was built, passed the parity tests and
// measured 108 us on [4096,16384] k = 50 against 86.5 us for the ring kernel with a CTA per row: a warp
// has one 4 KB tile in flight and nothing to do while it waits.  Not kept.
constexpr int kWarpRowCap = 256;
constexpr int kWarpRowMaxLen = 4096;

template <bool LARGEST, bool VEC, bool TWO /* k > 32: two values per lane enter the threshold */>
__global__ void __launch_bounds__(128, 8)
topk_warp_kernel(const float* __restrict__ in, TopkGeom g, float* __restrict__ out_val, long long* __restrict__ out_idx) {
    __shared__ unsigned long long cand_all[4][kWarpRowCap];
    __shared__ unsigned keys_all[4][64];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const long long r = (long long)blockIdx.x * 4 + warp;
    if (r >= g.rows) return;
    unsigned long long* cand = cand_all[warp];
    unsigned* keys = keys_all[warp];
    const float* row = topk_row(in, g, r);
    const int len = (int)g.len, k = (int)g.k;
    const int ntiles = (len + kWarpTile - 1) / kWarpTile;

    // element j (0..31) of this lane in tile t: float4 number u * 32 + lane, component c, j = 4u + c
    auto elem_of = [&](int t, int j) -> int { return t * kWarpTile + ((j >> 2) * 32 + lane) * 4 + (j & 3); };
    auto load_tile = [&](float4 (&v)[8], int t) {
        const int off = t * kWarpTile;
        if (VEC && off + kWarpTile <= len) {
            const float* p = row + off + lane * 4;
#pragma unroll
            for (int u = 0; u < 8; ++u) v[u] = ld_keep4(p + u * 128);
        } else {
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int e0 = off + (u * 32 + lane) * 4;
                float q[4];
#pragma unroll
                for (int c = 0; c < 4; ++c) q[c] = e0 + c < len ? *TPB_CK(&row[(long long)(e0 + c) * g.es]) : NAN;
                v[u] = make_float4(q[0], q[1], q[2], q[3]);
            }
        }
    };

    // ---- 1. the two best values per lane, compared as floats (-0.0 = +0.0 and NaN never better, as
    // the keys order them); a lane that saw fewer than two numbers keeps the worst value
    float4 v[8];
    const float worst = LARGEST ? -INFINITY : INFINITY;
    float f1 = worst, f2 = worst;
    for (int t = 0; t < ntiles; ++t) {
        load_tile(v, t);
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const float q[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                if (TWO) {
                    const bool g1 = LARGEST ? q[c] > f1 : q[c] < f1;
                    const bool g2 = LARGEST ? q[c] > f2 : q[c] < f2;
                    f2 = g1 ? f1 : (g2 ? q[c] : f2);
                    f1 = g1 ? q[c] : f1;
                } else {
                    f1 = LARGEST ? fmaxf(f1, q[c]) : fminf(f1, q[c]);   // a NaN operand is ignored
                }
            }
        }
    }
    // threshold key: the k-th best of the 32 best-per-lane values (k <= 32: a shuffle sort) or of all
    // 64 (rank counting, two slots per lane).  At least k elements of the row reach it, unless the
    // row has fewer than k numbers above the worst value -- then the count below falls short of k
    // and everything is taken.
    unsigned tkey = 0u;
    if (!TWO) {
        unsigned key = rank_key<LARGEST>(f1);
#pragma unroll
        for (int size = 2; size <= 32; size <<= 1) {
#pragma unroll
            for (int stride = size >> 1; stride > 0; stride >>= 1) {
                const unsigned o = __shfl_xor_sync(kFull, key, stride);
                const bool keep_max = ((lane & stride) == 0) == ((lane & size) == 0);
                key = keep_max ? (o > key ? o : key) : (o < key ? o : key);
            }
        }
        tkey = __shfl_sync(kFull, key, k - 1);      // descending: lane j holds the (j + 1)-th best
    } else {
        keys[lane] = rank_key<LARGEST>(f1);
        keys[32 + lane] = rank_key<LARGEST>(f2);
        __syncwarp();
        const unsigned a = keys[lane], b = keys[32 + lane];
        int ra = 0, rb = 0;   // how many of the 64 slots rank before this one (ties by slot number)
        for (int j = 0; j < 64; ++j) {
            const unsigned o = keys[j];
            ra += (o > a || (o == a && j < lane)) ? 1 : 0;
            rb += (o > b || (o == b && j < 32 + lane)) ? 1 : 0;
        }
        unsigned mine = ra == k - 1 ? a : (rb == k - 1 ? b : 0u);   // exactly one slot has rank k - 1
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) mine |= __shfl_xor_sync(kFull, mine, d);
        tkey = mine;
    }

    // ---- 2. the elements that reach the threshold: one float compare each (ties and both zeros pass,
    // NaN does not); a threshold key of 0 takes everything
    int n = 0;
    for (int attempt = 0; attempt < 2; ++attempt) {
        const bool all = tkey == 0u;
        const float tvf = key_value<LARGEST>(tkey);
        n = 0;
        for (int t = 0; t < ntiles; ++t) {
            if (ntiles > 1 || attempt > 0) load_tile(v, t);        // one tile: still in the registers
            unsigned mask = 0u;
            if (all || (LARGEST ? f1 >= tvf : f1 <= tvf)) {        // a lane whose best value misses has nothing
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const float q[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const bool pass = all || (LARGEST ? q[c] >= tvf : q[c] <= tvf);
                        mask |= (pass ? 1u : 0u) << (4 * u + c);
                    }
                }
            }
            // padding of a ragged last tile reads as NaN: only "take everything" can let it through
            if (all && (t + 1) * kWarpTile > len) {
#pragma unroll
                for (int j = 0; j < 32; ++j) if (elem_of(t, j) >= len) mask &= ~(1u << j);
            }
            const int cnt = __popc(mask);
            int incl = cnt;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const int o = __shfl_up_sync(kFull, incl, d);
                if (lane >= d) incl += o;
            }
            const int total = __shfl_sync(kFull, incl, 31);
            int pos = n + incl - cnt;
            if (n + total <= kWarpRowCap) {
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const float q[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const int j = 4 * u + c;
                        if (mask & (1u << j)) cand[pos++] = rank_word<LARGEST>(q[c], (unsigned)elem_of(t, j));
                    }
                }
            }
            n += total;
        }
        if (n >= k || all) break;
        tkey = 0u;      // fewer than k numbers above the worst value: NaN and the worst value belong to the answer
    }
    float* ov = out_val + r * k;
    long long* oi = out_idx + r * k;
    auto emit = [&](int j, unsigned long long w) {
        const unsigned idx = word_index(w);
        const unsigned key = (unsigned)(w >> 32);
        float val = key_value<LARGEST>(key);
        // the key folds -0.0 onto +0.0 and all NaNs onto one rank: those come from the row
        if (key == 0u || val == 0.0f) val = *TPB_CK(&row[(long long)idx * g.es]);
        *TPB_CK(&oi[j]) = (long long)idx;
        *TPB_CK(&ov[j]) = val;
    };
    if (n <= 32) {
        // ---- 3a. at most one word per lane: sorted with shuffles, no shared-memory traffic
        __syncwarp();
        unsigned long long w = lane < n ? cand[lane] : 0ull;
#pragma unroll
        for (int size = 2; size <= 32; size <<= 1) {
#pragma unroll
            for (int stride = size >> 1; stride > 0; stride >>= 1) {
                const unsigned long long o = __shfl_xor_sync(kFull, w, stride);
                const bool keep_max = ((lane & stride) == 0) == ((lane & size) == 0);
                w = keep_max ? (o > w ? o : w) : (o < w ? o : w);
            }
        }
        if (lane < k) emit(lane, w);
        return;
    }
    if (n <= kWarpRowCap) {
        // ---- 3. sort and write
        int N = 32;
        while (N < n) N <<= 1;
        for (int i = n + lane; i < N; i += 32) cand[i] = 0ull;
        __syncwarp();
        for (int size = 2; size <= N; size <<= 1) {
            for (int stride = size >> 1; stride > 0; stride >>= 1) {
                for (int q = lane; q < (N >> 1); q += 32) {
                    const int lo = ((q & ~(stride - 1)) << 1) | (q & (stride - 1));
                    const int hi = lo | stride;
                    const bool desc = (lo & size) == 0;
                    const unsigned long long x = cand[lo], y = cand[hi];
                    if ((x < y) == desc) { cand[lo] = y; cand[hi] = x; }
                }
                __syncwarp();
            }
        }
        for (int j = lane; j < k; j += 32) emit(j, cand[j]);
        return;
    }
    // ---- selection for rows with long runs of equal values: k times the best word below the last
    unsigned long long prev = ~0ull;
    for (int j = 0; j < k; ++j) {
        unsigned long long best = 0ull;
        for (int t = 0; t < ntiles; ++t) {
            load_tile(v, t);
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const float q[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const int e = elem_of(t, 4 * u + c);
                    if (e < len) {
                        const unsigned long long w = rank_word<LARGEST>(q[c], (unsigned)e);
                        if (w < prev && w > best) best = w;
                    }
                }
            }
        }
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) {
            const unsigned long long o = __shfl_xor_sync(kFull, best, d);
            best = o > best ? o : best;
        }
        if (lane == 0) emit(j, best);
        prev = best;
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
            skey[i] = rank_key<LARGEST>(*TPB_CK(&cv[i]));
            sidx[i] = *TPB_CK(&ci[i]) + (list_off ? *TPB_CK(&list_off[i / list_len]) : 0LL);
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
        *TPB_CK(&out_idx[j]) = sidx[j];
        *TPB_CK(&out_val[j]) = *TPB_CK(&cv[sslot[j]]);
    }
}

__device__ __forceinline__ int pow2_ceil_dev(int v) { return v <= 1 ? 1 : 1 << (32 - __clz(v - 1)); }

}  // namespace tpb

#undef TPB_FILE_ID
#define TPB_FILE_ID 3
#include "topk_select.cuh"
#undef TPB_FILE_ID
#define TPB_FILE_ID 2

namespace tpb {

// ------------------------------------------------------------------ planner ----------------
enum TopkPath { TK_NONE, TK_SORTROW, TK_STREAM, TK_SMALLK, TK_WARPROW };

struct TopkPlan {
    TopkPath path = TK_NONE;
    TopkGeom g{};
    bool vec = false;
    int N = 0;            // sort size of the sort-row path
    int mergeN = 0;       // sort size of the slice merge (S > 1)
    size_t ws_bytes = 0;  // slice survivors of the scanning kernels (S > 1); the select path needs none
    long long out_numel = 0;
    // select path (topk_select_kernel first, `path` as the second launch for flagged rows)
    bool select = false;
    SelGeom sel{};
    int sel_warps = 16;
};

// Smallest rank r with P(Poisson(mu) >= r) <= eps.
static int poisson_rank(double mu, double eps) {
    double pmf = std::exp(-mu), cdf = 0.0;   // pmf = P(X = i)
    for (int i = 0; i < 4096; ++i) {
        if (1.0 - cdf <= eps) return i < 1 ? 1 : i;   // 1 - cdf = P(X >= i)
        cdf += pmf;
        pmf *= mu / (double)(i + 1);
    }
    return 4096;
}

// Does the sampled-threshold kernel apply, and with which geometry?  (k, row length, rows only:
// the values are never looked at on the host.)
//   candidate buffer   6 k words (4096 .. 8192): the expected number of candidates is 2 to 3 k, and on
//                      tie-heavy rows whole classes of equal values are candidates together
//   CTA width          16 warps wherever a slice holds six rounds of tiles for them.  Measured on
//                      [512, 2^20], k = 1024: 512 CTAs of 16 warps in two waves 358 us, 512 CTAs of
//                      8 warps in one wave 444 us (an SM moves 46 GB/s with two 16-warp CTAs and 38 GB/s
//                      with three or four 8-warp CTAs); [256, 151936], k = 50: 32.1 against 38.6 us
//   CTAs per row       1, 2, 4 or 8 (a cluster), as many as one wave of CTAs on the GPU holds
//   sample             1, 2 or 4 tiles per warp: the smallest sample whose threshold is expected to let
//                      at most 40 % of the buffer through
static bool plan_select(long long rows, long long len, long long k, int sms, TopkPlan* pl) {
    int on = 1;
    if (env_int("TPB200_TOPK_SELECT", &on) && on == 0) return false;
    if (k < 1 || k > kMaxStreamK || len < 32 * 1024 || rows > 0x3fffffffLL / kSelMaxCluster) return false;
    // k <= 64 with enough rows to fill the GPU on their own: the ring kernel (one CTA per row, no
    // cluster, 9 KB of shared memory) is as fast or faster -- measured on [256,151936], k = 50: 30.5 us
    // against 30.7 us (two CTAs per row) and 32.5-34.4 us (one); on [512, 2^20], k = 64: 304 against 310 us
    if (k <= kSmallK && rows * 4 >= (long long)sms * 2 * 3 && !(env_int("TPB200_TOPK_SELECT", &on) && on == 2)) return false;
    const long long tiles = len / kWarpTile;
    const int cap = (int)std::min<long long>(8192, std::max<long long>(4096, round_up(6 * k, 256)));
    const size_t smem = (size_t)cap * 8 + 4096;     // per CTA, with the static part
    auto per_sm = [&](int nw) {
        const int by_threads = nw == 4 ? 7 : (nw == 8 ? 4 : 2);
        return (int)std::min<long long>(by_threads, (long long)(227 * 1024) / (long long)smem);
    };
    int nw = tiles >= 6LL * 16 ? 16 : (tiles >= 6LL * 8 ? 8 : 4);
    int fw = 0;
    if (env_int("TPB200_SEL_WARPS", &fw) && (fw == 4 || fw == 8 || fw == 16)) nw = fw;
    if (per_sm(nw) < 1) return false;
    const long long slots = (long long)sms * per_sm(nw);
    int S = 1;
    while (S < kSelMaxCluster && rows * (2LL * S) <= slots && tiles / (2LL * S) >= 6LL * nw) S *= 2;
    int fs = 0;
    if (env_int("TPB200_SEL_SLICES", &fs) && (fs == 1 || fs == 2 || fs == 4 || fs == 8)) S = fs;
    const long long slice_tiles = tiles / S;
    int fr = 0, ft = 0;
    const bool forced_rank = env_int("TPB200_SEL_RANK", &fr) && fr >= 1;
    const bool forced_tpw = env_int("TPB200_SEL_TPW", &ft) && (ft == 1 || ft == 2 || ft == 4);
    int tpw = 0, r = 0;
    for (int t : {1, 2, 4}) {
        if (forced_tpw && t != ft) continue;
        if ((long long)(t + 1) * nw * 3 > slice_tiles) break;        // sample at most a third of the slice
        const double m = (double)t * nw * kWarpTile;                // sampled elements per CTA
        const double mu = (double)k * m / (double)len;               // of which among the row's k best, on average
        const int rr = forced_rank ? fr : poisson_rank(mu, 1e-7);
        if (rr > 96) continue;
        const double expect = (double)rr * (double)len / m;          // candidates per row, values all distinct
        tpw = t;
        r = rr;
        if (expect <= 0.4 * cap) break;
    }
    if (tpw == 0) return false;
    if (!forced_rank && (double)r * (double)len / ((double)tpw * nw * kWarpTile) > 0.7 * cap) return false;
    SelGeom& sg = pl->sel;
    sg.S = S;
    sg.r = r;
    sg.cap = cap;
    sg.tpw = tpw;
    sg.prefetch = 0;
    env_int("TPB200_SEL_PREFETCH", &sg.prefetch);
    sg.inplace = 0;
    env_int("TPB200_SEL_INPLACE", &sg.inplace);
    sg.trigger = 1;
    sg.chunk = round_up(ceil_div(len, S), 4);
    // geometry of the scan that redoes a row inside the kernel (the rendezvous kernel's, one slice)
    sg.fb_B = pow2_ceil(std::max<long long>(4 * k, 1024));
    sg.fb_soft = (int)std::min<long long>(sg.fb_B / 2, std::max<long long>(320, 3 * k));
    pl->sel_warps = nw;
    return true;
}

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

    const char* force = env_str("TPB200_FORCE_TOPK");  // "sort" | "stream"
    const bool force_sort = force && std::string(force) == "sort";
    const bool force_stream = force && std::string(force) == "stream";

    if (len <= kWarpRowMaxLen && k <= 64 && !force_sort && !force_stream) {
        if (ceil_div(rows, 4) > 0x7fffffffLL) return fail(TPB200_ERR_UNSUPPORTED, "too many rows for one launch");
        pl->path = TK_WARPROW;      // a warp per row, one launch, no scratch
        return TPB200_OK;
    }
    if ((len <= 4096 && !force_stream) || k > kMaxStreamK || (force_sort && len <= kMaxSortRow)) {
        if (len > kMaxSortRow)
            return fail(TPB200_ERR_UNSUPPORTED, "k > %d is only supported on rows of at most %d elements", kMaxStreamK, kMaxSortRow);
        pl->path = TK_SORTROW;
        pl->N = std::max(2, pow2_ceil(len));
        return TPB200_OK;
    }
    const int sms = sm_count();
    // rows ride on grid.x together with the slices: 2^31 - 1 CTAs per launch
    auto grid_ok = [&](long long S) { return rows <= 0x7fffffffLL / std::max(1LL, S); };
    auto finish = [&]() {
        pl->select = plan_select(rows, len, k, sms, pl);
        if (pl->select) return TPB200_OK;       // one kernel, no scratch
        if (g.S > 1) {
            pl->mergeN = std::max(2, pow2_ceil((long long)g.S * k));
            pl->ws_bytes = (size_t)rows * g.S * k * sizeof(unsigned long long);
        }
        return TPB200_OK;
    };
    int smallk_on = 1;
    env_int("TPB200_TOPK_SMALLK", &smallk_on);   // 0: the general kernel for every k
    if (k <= kSmallK && smallk_on != 0) {
        // barrier-free ring kernel.  CTA width: 16 warps for long rows (one bootstrap and one final
        // step per row, no merge kernel; measured on [256,151936], k = 50: 30.4 us against 38.3 us
        // for 8 warps, 39.5 us for two 8-warp slices and 48.1 us for four 4-warp slices per row),
        // narrower CTAs for short rows; slices only where the rows alone cannot fill the GPU
        pl->path = TK_SMALLK;
        g.B = kRing;
        g.soft = kChunk;
        g.warps = len >= 64 * 1024 ? 16 : (len >= 16 * 1024 ? 8 : 4);
        int fw = 0;
        if (env_int("TPB200_TOPK_WARPS", &fw)) g.warps = fw == 16 ? 16 : (fw == 8 ? 8 : 4);
        const int per_sm = g.warps == 4 ? 7 : (g.warps == 8 ? 4 : 2);
        long long want = std::max(1LL, (long long)sms * per_sm / rows);
        long long most = std::max(1LL, len / (8LL * g.warps * kWarpTile));
        // the merge kernel sorts S * k words in shared memory
        long long cap = std::max(1LL, (long long)kMaxSortRow / k);
        long long S = std::min(std::min(want, most), cap);
        int fs = 0;
        if (env_int("TPB200_TOPK_SLICES", &fs)) S = std::max(1LL, std::min(std::min((long long)fs, cap), len / ((long long)g.warps * kWarpTile)));
        g.chunk = round_up(ceil_div(len, S), 4);
        g.S = (int)ceil_div(len, g.chunk);
        // the last slice must still hold one tile per warp for the bootstrap
        while (g.S > 1 && len - (long long)(g.S - 1) * g.chunk < (long long)g.warps * kWarpTile) {
            --S;
            g.chunk = round_up(ceil_div(len, S), 4);
            g.S = (int)ceil_div(len, g.chunk);
        }
        if (len < (long long)g.warps * kWarpTile) { g.warps = 4; }   // len > 4096 here, so four tiles exist
        if (!grid_ok(g.S)) return fail(TPB200_ERR_UNSUPPORTED, "too many rows for one launch");
        return finish();
    }
    pl->path = TK_STREAM;
    g.B = pow2_ceil(std::max<long long>(4 * k, 1024));
    // first cut early: handling a candidate costs far more than skipping an element, and only a cut
    // tightens the threshold (measured on [256,151936], k = 50: 320 words beats 160 and 1024)
    g.soft = (int)std::min<long long>(g.B / 2, std::max<long long>(320, 3 * k));
    int fb = 0, fso = 0, fw = 0;
    if (env_int("TPB200_TOPK_B", &fb)) g.B = std::max(g.B, pow2_ceil(fb));
    if (env_int("TPB200_TOPK_SOFT", &fso)) g.soft = std::min(g.B - 1, std::max(fso, (int)k + 1));
    // CTA width: 16 warps for long rows (half as many bootstraps / cuts as two 8-warp slices and,
    // with one CTA per row, no merge kernel), 8 warps for rows below 64 K elements.
    g.warps = len >= 64 * 1024 ? 16 : 8;
    if (env_int("TPB200_TOPK_WARPS", &fw)) g.warps = fw == 16 ? 16 : 8;
    // slices: fill the CTA slots of the GPU once, never overshoot them; each slice at least eight
    // rounds of all warps and at least 8k long
    const int slots = sms * (g.warps == 16 ? 2 : 4);
    long long want = std::max(1LL, (long long)slots / rows);
    long long most = std::max(1LL, len / std::max<long long>(8LL * g.warps * kWarpTile, 8 * k));
    long long cap = std::max(1LL, (long long)kMaxSortRow / k);
    // every slice of a large-k row pays its own cuts towards k: measured on [64..256, 2^20], k = 1024,
    // two slices per row are the most that still pay off
    if (k > 256) want = std::min(want, 2LL);
    long long S = std::max(1LL, std::min(std::min(want, most), cap));
    int fs = 0;
    if (env_int("TPB200_TOPK_SLICES", &fs)) S = std::max(1LL, std::min((long long)fs, cap));
    g.chunk = round_up(ceil_div(len, S), 4);
    g.S = (int)ceil_div(len, g.chunk);
    if (!grid_ok(g.S)) return fail(TPB200_ERR_UNSUPPORTED, "too many rows for one launch");
    return finish();
}

template <class K>
static int allow_smem(K kernel, size_t bytes) {
    if (bytes + 8192 > 48 * 1024) {   // static shared memory counts against the 48 KB default too
        TPB_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
    }
    return TPB200_OK;
}

template <bool LARGEST>
static int select_launch(const TopkPlan& pl, const float* in, float* ov, long long* oi, cudaStream_t st) {
    const TopkGeom& g = pl.g;
    SelGeom sg = pl.sel;
    sg.trigger = dependent_launch_on() ? 1 : 0;
    const size_t sm = std::max((size_t)sg.cap * 8, (size_t)sg.fb_B * 12);
    const unsigned grid = (unsigned)(g.rows * sg.S);
    const int nw = pl.sel_warps;
    int* status = device_status_word();
    cudaError_t e = cudaSuccess;
#define TPB_LAUNCH_SELECT(V, W)                                                                           \
    do {                                                                                                  \
        int rc = allow_smem(topk_select_kernel<LARGEST, V, W>, sm);                                       \
        if (rc) return rc;                                                                                \
        e = launch_ex(topk_select_kernel<LARGEST, V, W>, dim3(grid), W * 32, sm, st, sg.S, sg.trigger != 0, in, g, sg, ov, oi, status); \
    } while (0)
    if (pl.vec) { if (nw == 16) TPB_LAUNCH_SELECT(true, 16); else if (nw == 8) TPB_LAUNCH_SELECT(true, 8); else TPB_LAUNCH_SELECT(true, 4); }
    else        { if (nw == 16) TPB_LAUNCH_SELECT(false, 16); else if (nw == 8) TPB_LAUNCH_SELECT(false, 8); else TPB_LAUNCH_SELECT(false, 4); }
#undef TPB_LAUNCH_SELECT
    if (e != cudaSuccess) return cuda_fail(e, "topk_select_kernel");
    return TPB200_OK;
}

template <bool LARGEST>
static int topk_launch(const TopkPlan& pl, const float* in, float* ov, long long* oi, void* ws,
                       cudaStream_t st) {
    const TopkGeom& g = pl.g;
    if (pl.path == TK_WARPROW) {
        const dim3 grid((unsigned)ceil_div(g.rows, 4));
        if (g.k > 32) {
            if (pl.vec) TPB_LAUNCH("topk_warp_kernel", (topk_warp_kernel<LARGEST, true, true>), grid, 128, 0, st, in, g, ov, oi);
            else        TPB_LAUNCH("topk_warp_kernel", (topk_warp_kernel<LARGEST, false, true>), grid, 128, 0, st, in, g, ov, oi);
        } else {
            if (pl.vec) TPB_LAUNCH("topk_warp_kernel", (topk_warp_kernel<LARGEST, true, false>), grid, 128, 0, st, in, g, ov, oi);
            else        TPB_LAUNCH("topk_warp_kernel", (topk_warp_kernel<LARGEST, false, false>), grid, 128, 0, st, in, g, ov, oi);
        }
        return TPB200_OK;
    }
    if (pl.path == TK_SORTROW) {
        size_t sm = (size_t)pl.N * 8;
        int rc = allow_smem(topk_sort_kernel<LARGEST, true>, sm);
        if (rc) return rc;
        int threads = std::min(kSortThreads, std::max(32, pl.N / 2));
        if (g.rows > 0x7fffffffLL) return fail(TPB200_ERR_UNSUPPORTED, "too many rows for one launch");
        TPB_LAUNCH("topk_sort_kernel", (topk_sort_kernel<LARGEST, true>), dim3((unsigned)g.rows), threads, sm, st, in, g,
                   (const unsigned long long*)nullptr, (int)g.len, pl.N, ov, oi);
        return TPB200_OK;
    }
    // long rows: the sampled-threshold kernel, which redoes the rows that fail its check itself
    if (pl.select) return select_launch<LARGEST>(pl, in, ov, oi, st);
    const bool dep = false;   // the scanning kernels launch the ordinary way
    const unsigned grid = (unsigned)(g.rows * g.S);
    unsigned long long* w = g.S > 1 ? (unsigned long long*)ws : nullptr;
    int* status = device_status_word();
    const int threads = g.warps * 32;
    cudaError_t e = cudaSuccess;
    if (pl.path == TK_SMALLK) {
#define TPB_LAUNCH_SMALLK(V, W) e = launch_ex(topk_smallk_kernel<LARGEST, V, W>, dim3(grid), threads, 0, st, 1, dep, in, g, w, ov, oi, status)
        if (pl.vec) {
            if (g.warps == 16) TPB_LAUNCH_SMALLK(true, 16); else if (g.warps == 8) TPB_LAUNCH_SMALLK(true, 8); else TPB_LAUNCH_SMALLK(true, 4);
        } else {
            if (g.warps == 16) TPB_LAUNCH_SMALLK(false, 16); else if (g.warps == 8) TPB_LAUNCH_SMALLK(false, 8); else TPB_LAUNCH_SMALLK(false, 4);
        }
#undef TPB_LAUNCH_SMALLK
        if (e != cudaSuccess) return cuda_fail(e, "topk_smallk_kernel");
    } else {
        const size_t sm = (size_t)g.B * 12;
#define TPB_LAUNCH_STREAM(V, W)                                                                          \
    do {                                                                                                 \
        int rc = allow_smem(topk_stream_kernel<LARGEST, V, W>, sm);                                      \
        if (rc) return rc;                                                                               \
        e = launch_ex(topk_stream_kernel<LARGEST, V, W>, dim3(grid), threads, sm, st, 1, dep, in, g, w, ov, oi, status); \
    } while (0)
        if (pl.vec) { if (g.warps == 16) TPB_LAUNCH_STREAM(true, 16); else TPB_LAUNCH_STREAM(true, 8); }
        else        { if (g.warps == 16) TPB_LAUNCH_STREAM(false, 16); else TPB_LAUNCH_STREAM(false, 8); }
#undef TPB_LAUNCH_STREAM
        if (e != cudaSuccess) return cuda_fail(e, "topk_stream_kernel");
    }
    if (g.S > 1) {
        size_t msm = (size_t)pl.mergeN * 8;
        int rc = allow_smem(topk_sort_kernel<LARGEST, false>, msm);
        if (rc) return rc;
        int mthreads = std::min(kSortThreads, std::max(32, pl.mergeN / 2));
        e = launch_ex(topk_sort_kernel<LARGEST, false>, dim3((unsigned)g.rows), mthreads, msm, st, 1, dep, in, g, (const unsigned long long*)w,
                      g.S * (int)g.k, pl.mergeN, ov, oi);
        if (e != cudaSuccess) return cuda_fail(e, "topk_sort_kernel(merge)");
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

#ifdef TPB200_TRACE
extern "C" int tpb200_debug_trace(long long* host, int n) {
    return (int)cudaMemcpyFromSymbol(host, tpb::g_sel_trace, sizeof(long long) * n);
}
extern "C" int tpb200_debug_trace_clear(void) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, tpb::g_sel_trace) != cudaSuccess) return 1;
    return (int)cudaMemset(p, 0, sizeof(tpb::g_sel_trace));
}
#endif

extern "C" int tpb200_topk_plan_info(int dtype, int ndim, const int64_t* sizes, const int64_t* strides,
                                     int dim, int64_t k, int64_t* info, int n_info) {
    if (dtype != TPB200_F32) return fail(TPB200_ERR_UNSUPPORTED, "only float32 input is supported (dtype code %d)", dtype);
    if (!info || n_info < 1) return fail(TPB200_ERR_INVALID, "info is NULL or empty");
    TopkPlan pl;
    int rc = topk_plan((const void*)16, ndim, sizes, strides, dim, k, &pl);
    if (rc) return rc;
    const int scan_launches = pl.path == TK_NONE ? 0 : 1 + (pl.path != TK_SORTROW && pl.g.S > 1 ? 1 : 0);
    const int launches = pl.select ? 1 : scan_launches;
    const int64_t v[TPB200_PLAN_INFO_FIELDS] = {
        (int64_t)pl.path, pl.g.S, pl.g.warps, pl.select ? 1 : 0, pl.select ? pl.sel.S : 0,
        pl.select ? pl.sel_warps : 0, pl.select ? pl.sel.r : 0, pl.select ? pl.sel.cap : 0, pl.select ? pl.sel.tpw : 0,
        launches, (int64_t)pl.ws_bytes};
    for (int i = 0; i < n_info && i < TPB200_PLAN_INFO_FIELDS; ++i) info[i] = v[i];
    return TPB200_OK;
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
    TPB_CHECK_RANGES(st, view_range(in, ndim, sizes, strides, 4), HostRange{out_val, (size_t)pl.out_numel * 4},
                     HostRange{out_idx, (size_t)pl.out_numel * 8}, HostRange{workspace, pl.ws_bytes});
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
    TPB_CHECK_RANGES(st, HostRange{cand_val, (size_t)n_cand * 4}, HostRange{cand_idx, (size_t)n_cand * 8},
                     HostRange{list_offsets, list_offsets ? (size_t)(n_cand / ll) * 8 : 0},
                     HostRange{out_val, (size_t)k * 4}, HostRange{out_idx, (size_t)k * 8});
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
