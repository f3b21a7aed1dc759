// One-pass top-k with a sampled threshold, for long rows: topk_select_kernel.
// Included by topk.cu after the rank-word and sort helpers.
//
// The two scanning kernels of topk.cu learn their threshold while they scan: it only rises when a
// cut has seen k candidates, so a row cannot be split over CTAs without every slice paying for its
// own k candidates, and the first part of every row is scanned with a weak threshold (k(1 + ln(n/k))
// candidates per row at best).  This kernel fixes the threshold BEFORE the scan, from a sample, and
// verifies it afterwards (the scheme of Floyd and Rivest's SELECT: sample, pick a pivot with a safety
// margin, partition, check):
//
//   1. sample     every warp of a CTA streams its first `tpw` 1024-element tiles of the CTA's slice
//                 and keeps one maximum per lane; the CTA's threshold key is the r-th largest of its
//                 lane maxima.  r is chosen on the host so that, for a row whose order carries no
//                 information about its values, fewer than k elements of the ROW reach that key with
//                 probability below 1e-7: the number of sampled elements among the row's k best is
//                 Poisson(mu), mu = k * sample / n, and r is the smallest rank with
//                 P(Poisson(mu) >= r) <= 1e-7.  (A lane maximum ranks at or below the element of the
//                 same rank, so the estimate errs towards more candidates.)  The loads of the first
//                 scan tile are already in flight while the threshold is worked out.
//   2. scan       one pass, no barrier, no cut: an element is a candidate iff its key reaches the
//                 threshold key (one float compare; ties of the threshold value are all taken, so the
//                 index order among them is decided later and exactly).  Candidates are rank words in
//                 the CTA's shared memory, one atomic each.  The sample tiles are scanned first, while
//                 they are still in L2.
//   3. merge      the S CTAs of a row are one thread-block cluster.  A CTA that has finished its
//                 slice reserves room in the candidate buffer of the cluster's first CTA with one
//                 remote atomic (from the top down, while the first CTA may still be filling it from
//                 the bottom up), copies its words there with plain remote stores and reports its
//                 threshold key; one cluster barrier later the first CTA holds the candidates of the
//                 row.  Every CTA took all elements at or above its own key, so the union holds every
//                 element at or above the LARGEST of these keys, T*.
//   4. verify     the first CTA cuts the candidates to the k best, sorted.  The result is exact iff
//                 no buffer overflowed and the k-th best candidate has a key of at least T*: then at
//                 least k elements reach T*, all of them are candidates, and everything that is not a
//                 candidate ranks below them.  Otherwise the same CTA scans the row again the way
//                 topk_stream_kernel does (stream_body: a threshold learnt from cuts, no assumption).
//                 Rows whose beginning says nothing about the rest (sorted rows, all-equal rows, rows
//                 with fewer than k numbers) go that way; they cost a second pass, never a wrong
//                 answer, and no second launch.
//
// Splitting a row is cheap here (the threshold does not depend on the scan), so the planner picks
// CTA width and CTAs per row such that ONE wave of equal CTAs fills the GPU: co-resident CTAs share
// HBM bandwidth by their loads in flight, so equal CTAs finish together.  No TMA, no multicast: the
// cluster is used for its barrier and for remote shared-memory atomics and stores only.
#pragma once

#include <cooperative_groups.h>

namespace tpb {

namespace cg = cooperative_groups;

// Development builds (-DTPB200_TRACE) stamp the phases of every CTA with %globaltimer; the library
// then exports tpb200_debug_trace() to read the stamps back.  Ordinary builds compile none of it.
#ifdef TPB200_TRACE
constexpr int kTraceCtas = 4096, kTraceSlots = 16;
__device__ long long g_sel_trace[kTraceCtas * kTraceSlots];
__device__ __forceinline__ long long sel_now() { long long t; asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t)); return t; }
#define TPB_STAMP(i) do { if (threadIdx.x == 0) g_sel_trace[(blockIdx.x % kTraceCtas) * kTraceSlots + (i)] = sel_now(); } while (0)
#define TPB_NOTE(i, v) do { if (threadIdx.x == 0) g_sel_trace[(blockIdx.x % kTraceCtas) * kTraceSlots + (i)] = (long long)(v); } while (0)
#else
#define TPB_STAMP(i) do { } while (0)
#define TPB_NOTE(i, v) do { } while (0)
#endif

constexpr int kSelKeys = 128;        // lane-maximum keys that enter a CTA's estimate
constexpr int kSelMaxCluster = 8;    // portable cluster size

struct SelGeom {
    int S;           // CTAs (slices) per row = cluster size (1, 2, 4 or 8)
    int r;           // 1-based rank of the threshold key among a CTA's lane maxima
    int cap;         // candidate words of a CTA's buffer; also the limit per row
    int tpw;         // sample tiles per warp
    int prefetch;    // 1: hint the tiles after the first into L2 while the first is loaded
    int inplace;     // 1: the final cut always compacts in place (exercises that path; slower)
    int trigger;     // 1: launched as a dependent launch (programmatic dependent launch)
    int fb_B, fb_soft;  // buffer words and first-cut fill of the scan that redoes a failed row
    long long chunk; // slice length
};

struct SelShared {
    unsigned long long samp[128];   // pivot sample of the final cut, sorted descending
    unsigned long long raw[128];    // the same before sorting
    int wsum[32];                   // per-warp counts of the final cut's scan
    int hist[130], fill[130], start[130];   // sample sort of the final cut: bucket sizes, fill marks, first positions
    int bstar, taken;               // bucket of the k-th word; words in the buckets up to it
    unsigned bootk[kSelKeys];       // the warps' best lane maxima, as keys
    unsigned skeys[kSelKeys];       // the same, sorted descending
    unsigned tmax;                  // first CTA: largest threshold key reported by the other CTAs
    int cnt;                        // candidates reserved by this CTA (may exceed cap)
    int next;                       // next warp-tile of the slice
    int rem;                        // first CTA: words reserved by the other CTAs, from the top down
    int bad;                        // first CTA: a CTA of the row had no threshold or overflowed
    int base;                       // this CTA's reservation in the first CTA's buffer
    int tmp;
    StreamShared fb;                // control block of the scan that redoes a failed row
};

// The first CTA's last step: cut the n candidates in cand[0..n) to the k best, sorted, verify the
// k-th against the row's threshold key `tstar`, write the row.  Called by every thread of the CTA;
// returns true when the row must be redone.
//   n <= 256              every candidate counts the candidates above it: its rank is its output slot
//   otherwise             sample sort: 128 sorted sample words split the candidates into 129 buckets;
//                         the buckets that hold the k best are scattered behind the candidates and every
//                         word's rank inside its bucket gives its output slot (measured on 2900
//                         candidates, k = 1024: a 2048-word bitonic sort alone took 9 us of a 15 us cut)
//   no room for that      a pivot from the sample is tried until between k and two sort blocks of
//                         candidates reach it; those are compacted and sorted with the bitonic network
template <bool LARGEST, int NT>
__device__ bool sel_final(unsigned long long* cand, int n, int k, int cap, unsigned tstar, bool inplace, SelShared& sh,
                          const float* row, long long es, float* ov, long long* oi) {
    const int tid = threadIdx.x, lane = tid & 31;
    auto emit = [&](int j, unsigned long long w) {
        const unsigned idx = word_index(w);
        float val = key_value<LARGEST>((unsigned)(w >> 32));
        if (val == 0.0f) val = *TPB_CK(&row[(long long)idx * es]);   // the key folds -0.0 onto +0.0: the sign comes from the row
        *TPB_CK(&oi[j]) = (long long)idx;
        *TPB_CK(&ov[j]) = val;
    };
    if (tid == 0) sh.tmp = 0;
    __syncthreads();
    if (n <= 256) {
        // P threads share a candidate: each counts over its part of the list (whole warps take part,
        // so the shuffles are safe; a thread past the list works on word 0 and writes nothing)
        constexpr int P = NT >= 512 ? 2 : 1;
        const int step = (n + P - 1) / P;
        for (int i0 = 0; i0 < n; i0 += NT / P) {
            const int i = i0 + tid / P, part = tid % P;
            const unsigned long long w = i < n ? cand[i] : 0ull;
            int rank = 0;
            const int j1 = (part + 1) * step < n ? (part + 1) * step : n;
#pragma unroll 4
            for (int j = part * step; j < j1; ++j) rank += cand[j] > w ? 1 : 0;
            if (P >= 2) rank += __shfl_xor_sync(kFull, rank, 1);
            if (i < n && part == 0 && rank < k) {
                if (rank == k - 1 && (unsigned)(w >> 32) < tstar) sh.tmp = 1;
                emit(rank, w);
            }
        }
        __syncthreads();
        return sh.tmp != 0;
    }
    // ---- a sorted sample of 128 words (splitters), rank-sorted by P threads per word
    {
        constexpr int P = NT >= 512 ? 4 : (NT >= 256 ? 2 : 1);
        if (tid < 128) sh.raw[tid] = cand[(long long)tid * n / 128];
        __syncthreads();
        const int i = tid / P, part = tid % P;
        if (i < 128) {
            const unsigned long long my = sh.raw[i];
            int pos = 0;
#pragma unroll 8
            for (int j = part * (128 / P); j < (part + 1) * (128 / P); ++j) pos += sh.raw[j] > my ? 1 : 0;
            if (P >= 2) pos += __shfl_xor_sync(kFull, pos, 1);
            if (P >= 4) pos += __shfl_xor_sync(kFull, pos, 2);
            if (part == 0) sh.samp[pos] = my;    // the words of a row are distinct: no two share a rank
        }
        for (int j = tid; j < 130; j += NT) { sh.hist[j] = 0; sh.fill[j] = 0; }
        __syncthreads();
    }
    TPB_STAMP(10);
    // ---- sample sort of the words that can reach the output.  Bucket of a word = number of
    // splitters above it (0 .. 128); buckets are walked from the best down until they hold k words;
    // those words are scattered bucket by bucket behind the candidates, and a word's rank inside its
    // bucket (a scan of some twenty words) then gives its final position: it is written straight to
    // the output.  No sort network at all.
    // four words at a time: the seven steps of the four binary searches interleave, so that a thread
    // has four shared-memory loads in flight instead of one
    auto bucket_of4 = [&](const unsigned long long (&w)[4], int (&b)[4]) {
        int lo[4] = {0, 0, 0, 0}, hi[4] = {128, 128, 128, 128};
#pragma unroll
        for (int step = 0; step < 7; ++step) {
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int mid = (lo[u] + hi[u]) >> 1;
                if (sh.samp[mid] > w[u]) lo[u] = mid + 1; else hi[u] = mid;
            }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) b[u] = lo[u];
    };
    if (!inplace) {
        for (int base = 0; base < n; base += 4 * NT) {
            unsigned long long w[4];
            int b[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) { const int i = base + u * NT + tid; w[u] = i < n ? cand[i] : 0ull; }
            bucket_of4(w, b);
#pragma unroll
            for (int u = 0; u < 4; ++u) if (base + u * NT + tid < n) atomicAdd(&sh.hist[b[u]], 1);
        }
        __syncthreads();
        if (tid < 32) {
            // exclusive prefix over the 129 buckets (five per lane) and the bucket in which the k-th word lies
            int h[5], sum = 0;
#pragma unroll
            for (int e = 0; e < 5; ++e) { const int bb = tid * 5 + e; h[e] = bb < 129 ? sh.hist[bb] : 0; sum += h[e]; }
            int incl = sum;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) { const int t = __shfl_up_sync(kFull, incl, d); if (tid >= d) incl += t; }
            int run = incl - sum;
#pragma unroll
            for (int e = 0; e < 5; ++e) {
                const int bb = tid * 5 + e;
                if (bb < 129) {
                    sh.start[bb] = run;
                    if (run < k && run + h[e] >= k) { sh.bstar = bb; sh.taken = run + h[e]; }
                }
                run += h[e];
            }
        }
        __syncthreads();
        const int bstar = sh.bstar, T = sh.taken;
        TPB_STAMP(11);
        if (n + T <= cap) {
            unsigned long long* tmp = cand + n;
            for (int base = 0; base < n; base += 4 * NT) {
                unsigned long long w[4];
                int b[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) { const int i = base + u * NT + tid; w[u] = i < n ? cand[i] : 0ull; }
                bucket_of4(w, b);
#pragma unroll
                for (int u = 0; u < 4; ++u)
                    if (base + u * NT + tid < n && b[u] <= bstar) tmp[sh.start[b[u]] + atomicAdd(&sh.fill[b[u]], 1)] = w[u];
            }
            __syncthreads();
            TPB_STAMP(12);
            TPB_NOTE(14, T);
            for (int base = 0; base < T; base += 4 * NT) {
                unsigned long long w[4];
                int b[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) { const int p = base + u * NT + tid; w[u] = p < T ? tmp[p] : 0ull; }
                bucket_of4(w, b);
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    if (base + u * NT + tid >= T) continue;
                    const int s0 = sh.start[b[u]], s1 = s0 + sh.hist[b[u]];
                    int pos = s0;
#pragma unroll 4
                    for (int q = s0; q < s1; ++q) pos += tmp[q] > w[u] ? 1 : 0;
                    if (pos < k) {
                        if (pos == k - 1 && (unsigned)(w[u] >> 32) < tstar) sh.tmp = 1;
                        emit(pos, w[u]);
                    }
                }
            }
            __syncthreads();
            TPB_STAMP(13);
            return sh.tmp != 0;
        }
        // the bucket of the k-th word is too large for the room behind the candidates (or the buffer is
        // nearly full): fall through to the pivot cut below, which works in place
    }
    const int Nk = pow2_ceil_dev(k);
    int m = n;
    unsigned long long* arr = cand;       // where the words to sort end up
    if (!(pow2_ceil_dev(n) <= 2 * Nk && pow2_ceil_dev(n) <= cap)) {
        const int most = 2 * Nk < cap ? 2 * Nk : cap;
        // sample rank whose pivot is expected to keep about 1.19 k + 24 words
        int q = (int)(((long long)128 * (k + (k >> 3) + (k >> 4) + 24) + n - 1) / n) + 1;
        bool ok = false;
        unsigned long long pivot = 0ull;
        int excl = 0;
        for (int attempt = 0; attempt < 4 && q <= 127; ++attempt, q += 6) {
            pivot = sh.samp[q];
            // thread t counts over the words t, t + NT, ...; an exclusive scan of the counts gives
            // every thread the place of its words among those that are kept
            int c = 0;
            for (int i = tid; i < n; i += NT) c += cand[i] >= pivot ? 1 : 0;
            int incl = c;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const int t = __shfl_up_sync(kFull, incl, d);
                if (lane >= d) incl += t;
            }
            if (lane == 31) sh.wsum[tid >> 5] = incl;
            __syncthreads();
            int woff = 0, total = 0;
#pragma unroll
            for (int w = 0; w < NT / 32; ++w) {
                const int v = sh.wsum[w];
                woff += w < (tid >> 5) ? v : 0;
                total += v;
            }
            __syncthreads();
            excl = woff + incl - c;
            if (total >= k && total <= most) { ok = true; m = total; break; }
        }
        TPB_STAMP(11);
        if (!ok) {
            if (pow2_ceil_dev(n) > cap) return true;   // no pivot fits and no room to sort everything: redo
        } else if (n + most <= cap) {
            // room behind the candidates: every thread copies its kept words to its place there
            arr = cand + n;
            for (int i = tid; i < n; i += NT) {
                const unsigned long long w = cand[i];
                if (w >= pivot) arr[excl++] = w;
            }
            __syncthreads();
        } else {
            // no room: compact to the front in place.  A word only ever moves to a lower position, and
            // a batch is read completely before any of it is written
            for (int base = 0; base < n; base += NT) {
                const int i = base + tid;
                const unsigned long long w = i < n ? cand[i] : 0ull;
                const bool keep = w >= pivot;   // pivot > 0, so padding never passes
                const unsigned bal = __ballot_sync(kFull, keep);
                int wb = 0;
                __syncthreads();
                if (lane == 0 && bal) wb = atomicAdd(&sh.tmp, __popc(bal));
                wb = __shfl_sync(kFull, wb, 0);
                if (keep) cand[wb + __popc(bal & ((1u << lane) - 1u))] = w;
            }
            __syncthreads();
        }
    }
    const int N = pow2_ceil_dev(m) < 2 ? 2 : pow2_ceil_dev(m);
    for (int i = m + tid; i < N; i += NT) arr[i] = 0ull;
    __syncthreads();
    TPB_STAMP(12);
    TPB_NOTE(14, m);
    bitonic_desc(arr, N, tid, NT);
    TPB_STAMP(13);
    if ((unsigned)(arr[k - 1] >> 32) < tstar) return true;
    for (int j = tid; j < k; j += NT) emit(j, arr[j]);
    return false;
}

template <bool LARGEST, bool VEC, int NW>
__global__ void __launch_bounds__(NW * 32, NW == 4 ? 7 : (NW == 8 ? 4 : 2))
topk_select_kernel(const float* __restrict__ in, TopkGeom g, SelGeom sg, float* __restrict__ out_val,
                   long long* __restrict__ out_idx, int* status) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    unsigned long long* cand = reinterpret_cast<unsigned long long*>(smem_raw);   // cap words
    __shared__ SelShared sh;
    constexpr int NT = NW * 32;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int S = sg.S;
    cg::cluster_group cluster = cg::this_cluster();
    const int c = S > 1 ? (int)cluster.block_rank() : 0;
    const long long r = (long long)(blockIdx.x / (unsigned)S);
    const float* row = topk_row(in, g, r);
    const long long begin = (long long)c * sg.chunk;
    long long len = g.len - begin;
    if (len > sg.chunk) len = sg.chunk;
    if (len < 0) len = 0;
    const float* slice = row + begin * g.es;
    const int ntiles = (int)((len + kWarpTile - 1) / kWarpTile);
    const int k = (int)g.k, cap = sg.cap;

    TPB_STAMP(0);
    if (tid == 0) { sh.tmax = 0u; sh.cnt = 0; sh.next = 0; sh.rem = 0; sh.bad = 0; sh.base = 0; sh.tmp = 0; }
    // The other CTAs of the row write to this CTA's shared memory at the end of their scan; they must
    // see it initialised.  Arrive at the cluster barrier now (the release orders the line above) and
    // wait for it only after the scan, when every CTA has long arrived: the barrier costs nothing.
    if (S > 1) asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    if (sg.trigger) {
        // launched as a dependent launch (an experiment switch, off by default): this kernel may have
        // started before the previous kernel of the stream has finished; nothing is read or written
        // before this point
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
        asm volatile("griddepcontrol.wait;" ::: "memory");
    }

    auto elem_off = [&](long long off, int j) -> long long { return off + ((j >> 2) * 32 + lane) * 4 + (j & 3); };
    // A tile in registers; elements past the end of the slice read as NaN (never a candidate).
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
                for (int q = 0; q < 4; ++q) t[q] = e0 + q < len ? ld_stream1(slice + (e0 + q) * g.es) : NAN;
                v[u] = make_float4(t[0], t[1], t[2], t[3]);
            }
        }
    };
    auto mask_of = [&](const float4 (&v)[8], float tvf) -> unsigned {
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
    // Every masked element is a candidate: it is read again by address (an L2 hit) and its rank
    // word is appended.  A reservation past the buffer is only counted; the row is then redone.
    auto append = [&](unsigned m, long long off) {
        while (m != 0u) {
            const int j = __ffs(m) - 1;
            m &= m - 1u;
            const long long e = elem_off(off, j);
            if (e < len) {
                const float xv = *TPB_CK(&slice[e * g.es]);
                const int pos = atomicAdd(&sh.cnt, 1);
                if (pos < cap) cand[pos] = rank_word<LARGEST>(xv, (unsigned)(begin + e));
            }
        }
    };

    // ---- 1. sample: one maximum per lane over this warp's first tpw tiles; nothing is kept
    float4 v[8];
    float mx = NAN;   // fmaxf / fminf ignore a NaN operand
    for (int t = 0; t < sg.tpw; ++t) {
        load_tile(v, (long long)(t * NW + warp) * kWarpTile);
        if (VEC && sg.prefetch == 1 && t == 0) {
            // this warp's later sample tiles and its first scan tile: asked into L2 behind the loads of
            // the first tile, so that the loads that follow one another below find them there
            for (int u = 1; u <= sg.tpw; ++u) {
                const long long o = (long long)(u * NW + warp) * kWarpTile;
                if (o + kWarpTile <= len) asm volatile("prefetch.global.L2 [%0];" ::"l"(slice + o + lane * 32));
            }
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            if (LARGEST) mx = fmaxf(fmaxf(mx, v[u].x), fmaxf(fmaxf(v[u].y, v[u].z), v[u].w));
            else         mx = fminf(fminf(mx, v[u].x), fminf(fminf(v[u].y, v[u].z), v[u].w));
        }
    }
    TPB_STAMP(1);
    // the first scan tile of this warp: its loads are in flight while the threshold is worked out
    const int first_scan = sg.tpw * NW;               // tiles [first_scan, first_scan + NW) are taken here
    const long long off_b = (long long)(first_scan + warp) * kWarpTile;
    load_tile(v, off_b);
    if (VEC && sg.prefetch >= 2) {
        // experiment (TPB200_SEL_PREFETCH = 2 | 3): while the threshold is worked out nothing else is
        // loading; ask the tiles that the scan takes first after this one into L2 (one 128-byte line
        // per lane covers a tile).  Measured, k = 1024: [64, 2^20] 62.7 us without, 63.4 us with two
        // tiles per warp, 67.5 us with four; [512, 2^20] 356 / 354 / 353 us.  Off.
        const int per_warp = sg.prefetch == 2 ? 2 : 4;
        for (int u = 0; u < per_warp; ++u) {
            const long long o = (long long)(first_scan + NW + u * NW + warp) * kWarpTile;
            if (o + kWarpTile <= len) asm volatile("prefetch.global.L2 [%0];" ::"l"(slice + o + lane * 32));
        }
    }
    {
        unsigned key = rank_key<LARGEST>(mx);
#pragma unroll
        for (int size = 2; size <= 32; size <<= 1) {
#pragma unroll
            for (int stride = size >> 1; stride > 0; stride >>= 1) {
                const unsigned o = __shfl_xor_sync(kFull, key, stride);
                const bool keep_max = ((lane & stride) == 0) == ((lane & size) == 0);
                key = keep_max ? (o > key ? o : key) : (o < key ? o : key);
            }
        }
        constexpr int kShare = kSelKeys / NW;
        if (lane < kShare) sh.bootk[warp * kShare + lane] = key;
    }
    __syncthreads();
    {   // rank sort of the CTA's 128 keys (ties by position), P threads per key
        constexpr int P = NT >= 512 ? 4 : (NT >= 256 ? 2 : 1);
        const int i = tid / P, part = tid % P;
        if (i < kSelKeys) {
            const unsigned my = sh.bootk[i];
            int pos = 0;
#pragma unroll 8
            for (int j = part * (kSelKeys / P); j < (part + 1) * (kSelKeys / P); ++j) {
                const unsigned o = sh.bootk[j];
                pos += (o > my || (o == my && j < i)) ? 1 : 0;
            }
            if (P >= 2) pos += __shfl_xor_sync(kFull, pos, 1);
            if (P >= 4) pos += __shfl_xor_sync(kFull, pos, 2);
            if (part == 0) sh.skeys[pos] = my;
        }
    }
    __syncthreads();
    const unsigned tkey = sh.skeys[sg.r - 1];
    TPB_STAMP(2);
    // key 0 is the rank of NaN: the sample held fewer than r numbers, there is no float threshold
    const bool no_threshold = tkey == 0u;

    // ---- 2. scan: the tile already loaded, then the sample tiles (still in L2), then the rest
    if (!no_threshold) {
        const float tvf = key_value<LARGEST>(tkey);
        append(mask_of(v, tvf), off_b);
        for (;;) {
            int t = 0;
            if (lane == 0) t = atomicAdd(&sh.next, 1);
            t = __shfl_sync(kFull, t, 0);
            if (t >= first_scan) t += NW;
            if (t >= ntiles) break;
            const long long off = (long long)t * kWarpTile;
            unsigned m;
            {
                float4 w[8];
                load_tile(w, off);
                m = mask_of(w, tvf);
            }
            append(m, off);
        }
    }
    __syncthreads();
    if (S > 1) asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    TPB_STAMP(3);
    TPB_NOTE(8, sh.cnt);

    // ---- 3. merge the CTAs of the row into the first one
    int n = sh.cnt;
    bool bad = no_threshold || n > cap;
    if (n > cap) n = cap;
    unsigned tstar = tkey;
    if (S > 1) {
        if (c > 0) {
            if (tid == 0) {
                sh.base = atomicAdd(cluster.map_shared_rank(&sh.rem, 0u), n);
                atomicMax(cluster.map_shared_rank(&sh.tmax, 0u), tkey);
                if (bad) atomicOr(cluster.map_shared_rank(&sh.bad, 0u), 1);
            }
            __syncthreads();
            const int base = sh.base;
            if (base + n <= cap) {   // otherwise the row has overflowed; the first CTA sees it from `rem`
                unsigned long long* dst = cluster.map_shared_rank(cand, 0u) + (cap - base - n);
                for (int i = tid; i < n; i += NT) dst[i] = cand[i];
            }
            cluster.sync();   // the remote stores are complete and visible to the first CTA
            TPB_STAMP(4);
            return;
        }
        cluster.sync();
        const int rem = sh.rem;
        bad = bad || sh.bad != 0 || n + rem > cap;
        if (sh.tmax > tstar) tstar = sh.tmax;
        if (!bad) {
            // own words in [0, n), the others' in [cap - rem, cap): close the gap with words from the top
            const int gap = cap - rem - n;
            const int mv = rem < gap ? rem : gap;
            for (int i = tid; i < mv; i += NT) cand[n + i] = cand[cap - mv + i];
            n += rem;
        }
        __syncthreads();
        if (!bad) {
            // Every CTA took what reached ITS key; only words that reach the largest key T* can be in the
            // output if the check below holds (at least k of them), so the others are dropped here: the
            // cut works on fewer words.  In place: a word only moves to a lower position, and a batch is
            // read completely before any of it is written.
            const unsigned long long floor_word = (unsigned long long)tstar << 32;
            if (tid == 0) sh.tmp = 0;
            for (int base = 0; base < n; base += NT) {
                const int i = base + tid;
                const unsigned long long w = i < n ? cand[i] : 0ull;
                const bool keep = i < n && w >= floor_word;
                const unsigned bal = __ballot_sync(kFull, keep);
                int wb = 0;
                __syncthreads();
                if (lane == 0 && bal) wb = atomicAdd(&sh.tmp, __popc(bal));
                wb = __shfl_sync(kFull, wb, 0);
                if (keep) cand[wb + __popc(bal & ((1u << lane) - 1u))] = w;
            }
            __syncthreads();
            n = sh.tmp;
            __syncthreads();
        }
        TPB_STAMP(4);
    }

    // ---- 4. cut, verify, write
    bad = bad || n < k;
    TPB_NOTE(9, n);
    TPB_STAMP(5);
    if (!bad) bad = sel_final<LARGEST, NT>(cand, n, k, cap, tstar, sg.inplace != 0, sh, row, g.es, out_val + r * k, out_idx + r * k);
    TPB_STAMP(7);
    if (bad) {
        // The check failed (or a buffer overflowed, or the sample held too few numbers): this CTA scans
        // the whole row again the way topk_stream_kernel does, with a threshold that is learnt from
        // cuts and needs no assumption.  The other CTAs of the row have left.
        __syncthreads();
        TopkGeom fg = g;
        fg.S = 1;
        fg.chunk = g.len;
        fg.B = sg.fb_B;
        fg.soft = sg.fb_soft;
        fg.warps = NW;
        stream_body_call<LARGEST, VEC, NW>(row, fg, r, cand, sh.fb, out_val, out_idx, status);
    }
}

}  // namespace tpb
