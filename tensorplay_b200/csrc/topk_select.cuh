// One-pass top-k with a sampled threshold, for long rows: topk_select_kernel.
// Included by topk.cu after the rank-word, sort and cut helpers.
//
// The two streaming kernels of topk.cu learn their threshold while they scan: it only rises when a
// cut has seen k candidates, so a row cannot be split over CTAs without every slice paying for its
// own k candidates, and the first part of every row is scanned with a weak threshold (k(1 + ln(n/k))
// candidates per row at best).  This kernel fixes the threshold BEFORE the scan, from a sample, and
// verifies it afterwards (the scheme of Floyd and Rivest's SELECT: sample, pick a pivot with a safety
// margin, partition, check):
//
//   1. sample     every warp of the S CTAs of a row loads its first 1024-element tile and sorts its
//                 32 lane maxima; the CTA's best 128 are exchanged over distributed shared memory
//                 (the S CTAs of a row are one thread-block cluster) and every CTA finds the r-th
//                 largest key of the union.  r is chosen on the host so that, for a row whose order
//                 carries no information about its values, fewer than k elements reach that key with
//                 probability below 1e-7: the number of sampled elements among the row's k best is
//                 Poisson(mu), mu = k * sample / n, and r is the smallest rank with
//                 P(Poisson(mu) >= r) <= 1e-7.
//   2. scan       one pass, no barrier, no cut: an element is a candidate iff its key reaches the
//                 threshold key (one float compare; ties of the threshold value are all taken, so the
//                 index order among them is decided later and exactly).  Candidates are rank words in
//                 the CTA's shared memory, one atomic each.
//   3. merge      cluster barrier; the CTAs copy their candidates into the buffer of the cluster's
//                 first CTA through distributed shared memory (plain remote stores); that CTA cuts
//                 them to the k best, sorted, and writes the row's output.
//   4. verify     the result is exact iff at least k candidates were found and no buffer overflowed:
//                 every element outside the candidates ranks below all of them.  Otherwise the row is
//                 flagged and a second launch -- the scanning kernels of topk.cu, which need no
//                 assumption -- redoes exactly the flagged rows.  Rows whose beginning says nothing
//                 about the rest (sorted rows, all-equal rows, rows with fewer than k numbers) go
//                 that way; they cost a second pass, never a wrong answer.
//
// Splitting a row costs nothing here (the threshold does not depend on the scan), so the planner
// uses as many slices as fill the GPU: clusters of 2 to 8 CTAs per row.  No TMA, no multicast: the
// cluster is used for its barrier and for remote shared-memory loads and stores only.
#pragma once

#include <cooperative_groups.h>

namespace tpb {

namespace cg = cooperative_groups;

constexpr int kSelKeys = 128;        // lane-maximum keys that every CTA offers to the estimate
constexpr int kSelMaxCluster = 8;    // portable cluster size

struct SelGeom {
    int S;           // CTAs (slices) per row = cluster size (1, 2, 4 or 8)
    int r;           // 1-based rank of the threshold key among the sample's lane maxima
    int cap;         // candidate words per CTA buffer (power of two); also the limit per row
    int prefetch;    // tiles per warp hinted into L2 before the threshold is known
    int trigger;     // 1: let a dependent launch start early (programmatic dependent launch)
    long long chunk; // slice length
};

struct SelShared {
    StreamShared cs;                              // scratch of cut()
    unsigned bootk[kSelKeys];                     // the warps' best lane maxima, as keys
    unsigned skeys[kSelKeys];                     // the same, sorted descending; read by the cluster
    unsigned allk[kSelMaxCluster * kSelKeys];     // the sorted lists of all CTAs of the row
    unsigned tkey;                                // threshold key (0: no usable threshold)
    int cnt;                                      // candidates reserved by this CTA (may exceed cap)
    int next;                                     // next warp-tile of the slice
    int base, total, bad;                         // merge: offset in the first CTA's buffer, row total, verdict
};

// Entries of the descending list a[0..128) that are greater than / at least `key`.
__device__ __forceinline__ int sel_count_gt(const unsigned* a, unsigned key) {
    int lo = 0, hi = kSelKeys;
    while (lo < hi) { const int mid = (lo + hi) >> 1; if (a[mid] > key) lo = mid + 1; else hi = mid; }
    return lo;
}
__device__ __forceinline__ int sel_count_ge(const unsigned* a, unsigned key) {
    int lo = 0, hi = kSelKeys;
    while (lo < hi) { const int mid = (lo + hi) >> 1; if (a[mid] >= key) lo = mid + 1; else hi = mid; }
    return lo;
}

template <bool LARGEST, bool VEC, int NW>
__global__ void __launch_bounds__(NW * 32, NW == 4 ? 7 : (NW == 8 ? 4 : 2))
topk_select_kernel(const float* __restrict__ in, TopkGeom g, SelGeom sg, float* __restrict__ out_val,
                   long long* __restrict__ out_idx, int* __restrict__ fail) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    unsigned long long* cand = reinterpret_cast<unsigned long long*>(smem_raw);   // cap words
    unsigned long long* buf2 = cand + sg.cap;                                     // cap / 2 words (cut's partition target)
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

    if (tid == 0) { sh.tkey = 0u; sh.cnt = 0; sh.next = NW; sh.base = 0; sh.total = 0; sh.bad = 0; }
    if (sg.trigger) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

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
                const float xv = slice[e * g.es];
                const int pos = atomicAdd(&sh.cnt, 1);
                if (pos < cap) cand[pos] = rank_word<LARGEST>(xv, (unsigned)(begin + e));
            }
        }
    };

    // ---- 1. sample: this warp's first tile stays in registers until the threshold is known
    float4 v0[8];
    const long long off0 = (long long)warp * kWarpTile;
    load_tile(v0, off0);
    if (VEC) {
        // hint the tiles that this CTA scans next into L2 while the threshold is being found
        for (int i = 0; i < sg.prefetch; ++i) {
            const long long t = (long long)NW * (1 + i) + warp;
            if ((t + 1) * kWarpTile <= len) asm volatile("prefetch.global.L2 [%0];" ::"l"(slice + t * kWarpTile + lane * 32));
        }
    }
    {
        float mx = NAN;   // fmaxf / fminf ignore a NaN operand
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            if (LARGEST) mx = fmaxf(fmaxf(mx, v0[u].x), fmaxf(fmaxf(v0[u].y, v0[u].z), v0[u].w));
            else         mx = fminf(fminf(mx, v0[u].x), fminf(fminf(v0[u].y, v0[u].z), v0[u].w));
        }
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
    if (tid < kSelKeys) {   // rank sort of the CTA's 128 keys (ties by position)
        const unsigned my = sh.bootk[tid];
        int pos = 0;
        for (int i = 0; i < kSelKeys; ++i) {
            const unsigned o = sh.bootk[i];
            pos += (o > my || (o == my && i < tid)) ? 1 : 0;
        }
        sh.skeys[pos] = my;
    }
    __syncthreads();
    if (S > 1) {
        cluster.sync();
        for (int i = tid; i < S * kSelKeys; i += NT) {
            const unsigned* rk = cluster.map_shared_rank(sh.skeys, (unsigned)(i / kSelKeys));
            sh.allk[i] = rk[i % kSelKeys];
        }
        __syncthreads();
        for (int i = tid; i < S * kSelKeys; i += NT) {
            const unsigned my = sh.allk[i];
            int gt = 0, ge = 0;
            for (int l = 0; l < S; ++l) {
                gt += sel_count_gt(sh.allk + l * kSelKeys, my);
                ge += sel_count_ge(sh.allk + l * kSelKeys, my);
            }
            if (gt < sg.r && sg.r <= ge) sh.tkey = my;   // the same value from every writer
        }
    } else if (tid == 0) {
        sh.tkey = sh.skeys[sg.r - 1];
    }
    __syncthreads();
    const unsigned tkey = sh.tkey;
    // key 0 is the rank of NaN: the sample held fewer than r numbers, there is no float threshold
    const bool no_threshold = tkey == 0u;

    // ---- 2. scan
    if (!no_threshold) {
        const float tvf = key_value<LARGEST>(tkey);
        append(mask_of(v0, tvf), off0);
        for (;;) {
            int t = 0;
            if (lane == 0) t = atomicAdd(&sh.next, 1);
            t = __shfl_sync(kFull, t, 0);
            if (t >= ntiles) break;
            const long long off = (long long)t * kWarpTile;
            unsigned m;
            {
                float4 v[8];
                load_tile(v, off);
                m = mask_of(v, tvf);
            }
            append(m, off);
        }
    }
    __syncthreads();

    // ---- 3. merge the CTAs of the row into the first one
    int n = sh.cnt;
    bool bad = no_threshold || n > cap;
    if (n > cap) n = cap;
    if (S > 1) {
        cluster.sync();   // every CTA of the row has finished its scan
        if (tid == 0) {
            int base = 0, total = 0, over = 0;
            for (int q = 0; q < S; ++q) {
                int cn = *cluster.map_shared_rank(&sh.cnt, (unsigned)q);
                if (cn > cap) { over = 1; cn = cap; }
                if (q < c) base += cn;
                total += cn;
            }
            sh.base = base;
            sh.total = total;
            sh.bad = (over || total > cap) ? 1 : 0;
        }
        __syncthreads();
        bad = bad || sh.bad != 0;
        if (!bad && c > 0) {
            unsigned long long* dst = cluster.map_shared_rank(cand, 0u) + sh.base;
            for (int i = tid; i < n; i += NT) dst[i] = cand[i];
        }
        cluster.sync();   // remote stores done; nobody reads this CTA's shared memory any more
        if (c > 0) return;
        n = sh.total;
    }

    // ---- 4. verify; cut to the k best, sorted; write the row
    bad = bad || n < k;
    if (tid == 0) fail[r] = bad ? 1 : 0;
    if (bad) return;   // the second launch redoes this row
    if (tid == 0) sh.cs.cnt = n;
    __syncthreads();
    cut(cand, buf2, &sh.cs, cap, k, tid, NT, true);
    for (int j = tid; j < k; j += NT) {
        const unsigned long long w = cand[j];
        const unsigned idx = word_index(w);
        const unsigned key = (unsigned)(w >> 32);
        float val = key_value<LARGEST>(key);
        // the key folds -0.0 onto +0.0: the sign comes from the row
        if (val == 0.0f) val = row[(long long)idx * g.es];
        out_idx[r * k + j] = (long long)idx;
        out_val[r * k + j] = val;
    }
}

}  // namespace tpb
