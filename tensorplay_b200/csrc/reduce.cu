// Reductions (sum / mean / var / std / max / min / argmax / argmin and the fused value+index
// forms) for float32 tensors on sm_100a, behind tpb200_reduce and the sharded partial/combine
// entry points.  Replaces cuda::*_kernel of p10/src/backend/cuda/ReductionKernels.cu:54-382
// (one thread per row for argmax, cudnnReduceTensor for the rest, a 6-launch composition for var).
//
// Every kernel is HBM-bound: the input is read exactly once with 128-bit streaming loads, the
// strided view is consumed in place (no .contiguous() copy), and the arithmetic per element is a
// handful of instructions.  A host-side planner canonicalises (sizes, strides, reduce mask) into
// one of four kernel families:
//
//   ROW      the innermost reduced dim is contiguous: a row is `nseg` runs of `seglen` floats
//            - row_warp_kernel : one warp per row            (short rows, many rows)
//            - row_cta_kernel  : one CTA per row             (rows of a few KB .. a few hundred KB)
//            - row_split_kernel + finalize_kernel : S CTAs per row, fixed slices, then a
//              fixed-order combine of the S packed partials  (few very long rows, whole tensor)
//   COL      the innermost KEPT dim is contiguous, one reduced dim strides over it:
//            col_kernel (each thread owns 4 adjacent columns, 16-byte loads stay coalesced along
//            the kept dim) (+ col_finalize_kernel when the reduced dim is split over CTAs)
//   GENERIC  anything else (and empty reductions): one warp per output, div/mod addressing
//
// All combines run in a fixed order, so results are bit-reproducible run to run.
#define TPB_FILE_ID 1
#include "common.cuh"
#include "host_util.h"

#include <algorithm>
#include <atomic>
#include <cmath>
#include <mutex>
#include <string>
#include <vector>

namespace tpb {

// Development builds (-DTPB200_TRACE) stamp the whole-tensor path with %globaltimer: slot 0 earliest
// start and slot 1 latest end of the slice kernel's CTAs, slots 2..6 of the exchange kernel: start,
// own partials merged, record and flag published to every rank, every rank's flag seen, result
// written.  tpb200_debug_reduce_trace() reads them back.  Ordinary builds compile none of it.
#ifdef TPB200_TRACE
__device__ unsigned long long g_red_trace[8];
__device__ __forceinline__ unsigned long long red_now() { unsigned long long t; asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t)); return t; }
#define TPB_RED_STAMP(i) (g_red_trace[i] = red_now())
#define TPB_RED_STAMP_MIN(i) atomicMin(&g_red_trace[i], red_now())
#define TPB_RED_STAMP_MAX(i) atomicMax(&g_red_trace[i], red_now())
#else
#define TPB_RED_STAMP(i) do { } while (0)
#define TPB_RED_STAMP_MIN(i) do { } while (0)
#define TPB_RED_STAMP_MAX(i) do { } while (0)
#endif

// ------------------------------------------------------------------ geometry ---------------
struct RowGeom {
    long long rows;                      // number of outputs
    long long k1;                        // size of the inner kept dim (rows = k0 * k1)
    long long ks0, ks1;                  // element strides of the outer / inner kept dim
    long long nseg, seglen, seg_stride;  // one row = nseg runs of seglen contiguous floats
};

struct GenGeom {
    int nk, nr;
    long long ksize[TPB200_MAX_DIMS], kstride[TPB200_MAX_DIMS];
    long long rsize[TPB200_MAX_DIMS], rstride[TPB200_MAX_DIMS];
    long long outs, count;
};

__device__ __forceinline__ const float* row_base(const float* in, const RowGeom& g, long long r) {
    long long a = r / g.k1;
    long long b = r - a * g.k1;
    return in + a * g.ks0 + b * g.ks1;
}

template <class Acc>
__device__ __forceinline__ void add4(Acc& acc, const float4& v, long long b) {
    acc.add4(v.x, v.y, v.z, v.w, b, 1);
}

// ------------------------------------------------------------------ ROW: warp per row ------
template <class Acc, int UNROLL>
__device__ __forceinline__ void row_warp_body(const float* __restrict__ in, const RowGeom& g, const Epilogue& e,
                                              float* ov, long long* oi) {
    const int lane = threadIdx.x & 31;
    const long long r = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (r >= g.rows) return;
    // (A persistent grid walking the rows was measured on [4096,4096] -- 1024 CTAs of 4 warps = 6.9 per SM
    //  here, 12.5 us: 2 / 3 / 4 / 6 CTAs per SM 23.4 / 19.1 / 15.2 / 16.3 us, never better than a warp per
    //  row; and the loop alone cost the product 0.9 us.  Not kept.)
    const float* p = row_base(in, g, r);
    Acc acc;
    acc.init();
    for (long long s = 0; s < g.nseg; ++s)
        scan_contig<UNROLL>(acc, p + s * g.seg_stride, g.seglen, s * g.seglen, lane, 32);
    acc.finish_thread();
    warp_combine(acc);
    if (lane == 0) write_result(acc, e, (double)g.nseg * (double)g.seglen, ov, oi, r);
}
// Runs of fewer than 2048 floats: four loads in flight per lane, and whatever registers the compiler
// takes for 256 threads (48: short rows want warps, not registers -- [1048576, 64] and the variance of
// [65536, 1024] are 20-40 % slower with 72).
template <class Acc>
__global__ void __launch_bounds__(256)
row_warp_kernel(const float* __restrict__ in, RowGeom g, Epilogue e, float* ov, long long* oi) {
    row_warp_body<Acc, 4>(in, g, e, ov, oi);
}
// Runs of 2048 floats and more: eight loads in flight per lane and up to 72 registers (seven 4-warp CTAs
// per SM still fit).  At 48 the variance spilled and the others were squeezed: [4096,4096] var 12.9 ->
// 12.2 us, sum 12.2 -> 11.9 us; [2048,8192] 14.0 -> 12.4 us.
template <class Acc>
__global__ void __maxnreg__(72)
row_warp_long_kernel(const float* __restrict__ in, RowGeom g, Epilogue e, float* ov, long long* oi) {
    row_warp_body<Acc, 8>(in, g, e, ov, oi);
}

// ------------------------------------------------------------------ ROW: several rows per warp
// Contiguous rows of at most 256 floats: G = 4, 8 or 16 lanes share a row (a lane holds at most four
// float4), so a warp works on 8, 4 or 2 rows at once and all 32 lanes load.  One warp per 64-float row
// moved 0.96 TB/s on [1048576, 64]: half the lanes idle and five shuffle steps per 256 bytes.
template <class Acc, int G>
__global__ void __launch_bounds__(256)
row_group_kernel(const float* __restrict__ in, RowGeom g, Epilogue e, float* ov, long long* oi) {
    const int lane = threadIdx.x & 31, li = lane & (G - 1);
    const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const long long r = w * (32 / G) + lane / G;
    // every lane takes part in the shuffles; lanes of a row past the end work on nothing
    Acc acc;
    acc.init();
    if (r < g.rows) scan_contig<4>(acc, row_base(in, g, r), g.seglen, 0, li, G);
    acc.finish_thread();
#pragma unroll
    for (int d = G / 2; d > 0; d >>= 1) {
        Acc o = acc.shfl_down(d);
        acc.merge(o);
    }
    if (li == 0 && r < g.rows) write_result(acc, e, (double)g.seglen, ov, oi, r);
}

// ------------------------------------------------------------------ ROW: CTA per row -------
// tps = threads that share one run (power of two).  With several runs per row the CTA is a
// (tps x blockDim/tps) grid of threads: x walks along a run, y over runs, and loads of four
// different runs are issued together so a thread always has 64 bytes in flight.
// CTAs per SM that the register budget is cut for: three of 512 threads (40 registers) by default.
// The product gets 64 registers (two CTAs per SM): squeezed into 40 the compiler no longer kept the
// four loads of a step in flight together -- prod over dims (0,2) of [64,4096,512] 106.5 us with three
// CTAs per SM, 85.0 us with two.  The variance is the other way round (94.0 us with three, 107.6 us
// with two), the rest showed no difference.
template <class Acc> struct RowCtaBounds { static constexpr int kMinCtas = 3; };
template <> struct RowCtaBounds<ProdAcc> { static constexpr int kMinCtas = 2; };

template <class Acc>
__global__ void __launch_bounds__(512, RowCtaBounds<Acc>::kMinCtas)
row_cta_kernel(const float* __restrict__ in, RowGeom g, int tps, int vec_ok, Epilogue e, float* ov,
               long long* oi) {
    __shared__ Acc sm[32];
    const int tid = threadIdx.x, nthr = blockDim.x;
    const long long r = blockIdx.x;
    const float* p = row_base(in, g, r);
    Acc acc;
    acc.init();
    if (g.nseg == 1) {
        scan_contig<4>(acc, p, g.seglen, 0, tid, nthr);
    } else {
        const int tx = tid & (tps - 1);
        const int ty = tid / tps;
        const int ny = nthr / tps;
        const long long sv = g.seglen >> 2;
        if (vec_ok && sv <= tps) {
            for (long long s = ty; s < g.nseg; s += 4LL * ny) {
                float4 v[4];
                bool ok[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    long long ss = s + (long long)u * ny;
                    ok[u] = ss < g.nseg && tx < sv;
                    if (ok[u]) v[u] = ld_stream4(p + ss * g.seg_stride + 4 * tx);
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    long long ss = s + (long long)u * ny;
                    if (ok[u]) add4(acc, v[u], ss * g.seglen + 4 * tx);
                }
            }
        } else {
            for (long long s = ty; s < g.nseg; s += ny)
                scan_contig<2>(acc, p + s * g.seg_stride, g.seglen, s * g.seglen, tx, tps);
        }
    }
    acc.finish_thread();
    block_combine(acc, sm);
    if (tid == 0) write_result(acc, e, (double)g.nseg * (double)g.seglen, ov, oi, r);
}

// ------------------------------------------------------------------ ROW: split rows --------
// Pass 1: S CTAs per row, all resident at once.  CTA s of row r reduces the blocks s, s + S, s + 2S,
// ... of `sub` elements each to ONE packed partial: the CTAs of a row walk through it side by side
// and finish together, so there is one ramp and one tail per launch instead of one per wave of
// slices (measured on 2^28 elements: contiguous slices in four waves 163-169 us).  The
// assignment of blocks to CTAs and the order inside a thread are fixed, so results stay
// bit-reproducible; every thread still sees its elements in ascending position.
template <class Acc>
__global__ void __launch_bounds__(512)
row_split_kernel(const float* __restrict__ in, RowGeom g, long long sub, int S, Packed* ws) {
    __shared__ Acc sm[32];
    const int tid = threadIdx.x, nthr = blockDim.x;
    const long long s = blockIdx.x % (unsigned)S, r = blockIdx.x / (unsigned)S;
    if (tid == 0) TPB_RED_STAMP_MIN(0);
    const float* p = row_base(in, g, r);
    Acc acc;
    acc.init();
    for (long long b = s * sub; b < g.seglen; b += (long long)S * sub) {
        const long long len = g.seglen - b < sub ? g.seglen - b : sub;
        scan_contig<4>(acc, p + b, len, b, tid, nthr);
    }
    acc.finish_thread();
    block_combine(acc, sm);
    if (tid == 0) {
        acc.store(TPB_CK(&ws[r * S + s]));
        TPB_RED_STAMP_MAX(1);
    }
}

// Lane `lane` of a warp merges partials lane, lane + 32, ... of `ws` into r, in that order.  Up to 640
// partials (20 per lane) are loaded first and merged afterwards: with the load inside the merge loop
// every step waited for its own load (the variance's merge is too long for the compiler to unroll the
// loop: 8-9 us for 444 partials, against 1.4-2 us for the sum's 592).
template <class Acc>
__device__ __forceinline__ void merge_partials(Acc& r, const Packed* __restrict__ ws, int S, int lane) {
    constexpr int kPre = 20;
    if (S <= 32 * kPre) {
        Acc part[kPre];
#pragma unroll
        for (int u = 0; u < kPre; ++u) {
            const int q = lane + 32 * u;
            if (q < S) part[u].load(TPB_CK(&ws[q]));
        }
#pragma unroll
        for (int u = 0; u < kPre; ++u) {
            const int q = lane + 32 * u;
            if (q < S) r.merge(part[u]);
        }
    } else {
        for (int q = lane; q < S; q += 32) {
            Acc o;
            o.load(TPB_CK(&ws[q]));
            r.merge(o);
        }
    }
}

// Pass 2: one warp per row merges that row's S partials in a fixed order (lane l takes
// l, l+32, ..., then the lane tree).  Writes the finished result, or -- for the sharded path --
// one packed record whose position is shifted to the tensor-global index space.
template <class Acc>
__global__ void __launch_bounds__(128)
finalize_kernel(const Packed* __restrict__ ws, long long rows, int S, double count, Epilogue e,
                float* ov, long long* oi, Packed* packed_out, long long idx_offset) {
    const int lane = threadIdx.x & 31;
    const long long r = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (r >= rows) return;
    Acc acc;
    acc.init();
    acc.finish_thread();
    merge_partials(acc, ws + r * S, S, lane);
    warp_combine(acc);
    if (lane == 0) {
        if (packed_out) {
            Packed out;
            acc.store(&out);
            if (out.i0 != kNoIndex) out.i0 += idx_offset;
            *TPB_CK(&packed_out[r]) = out;
        } else {
            write_result(acc, e, count, ov, oi, r);
        }
    }
}

// ------------------------------------------------------------------ COL --------------------
// Input viewed as [O, L, I] with I contiguous and kept, L reduced.  blockIdx.x = tile + tiles*o,
// blockIdx.y = slice of L.  Thread (tx, ty) owns VEC adjacent columns and walks L with stride ny,
// four rows in flight.  Cross-ty combine is a fixed tree in shared memory.
template <class Acc, int VEC>
__global__ void __launch_bounds__(256)
col_kernel(const float* __restrict__ in, long long o_stride, long long L, long long l_stride,
           long long I, int tiles, int tx_n, long long lchunk, Packed* ws, Epilogue e, float* ov,
           long long* oi) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    Acc* sm = reinterpret_cast<Acc*>(smem_raw);
    const int tid = threadIdx.x, nthr = blockDim.x;
    const int tx = tid & (tx_n - 1), ty = tid / tx_n, ny = nthr / tx_n;
    const long long o = blockIdx.x / tiles;
    const int tile = (int)(blockIdx.x - o * tiles);
    const int s = blockIdx.y, S = gridDim.y;
    const long long i0 = ((long long)tile * tx_n + tx) * VEC;
    const bool active = i0 < I;
    const float* base = in + o * o_stride + i0;
    const long long l0 = (long long)s * lchunk;
    long long l1 = l0 + lchunk;
    if (l1 > L) l1 = L;

    Acc acc[VEC];
#pragma unroll
    for (int v = 0; v < VEC; ++v) acc[v].init();

    if (active) {
        for (long long l = l0 + ty; l < l1; l += 4LL * ny) {
            if (VEC == 4) {
                float4 x[4];
                bool ok[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    long long ll = l + (long long)u * ny;
                    ok[u] = ll < l1;
                    if (ok[u]) x[u] = ld_stream4(base + ll * l_stride);
                }
                if (ok[3]) {
                    // four rows of each of this thread's columns at once
                    acc[0].add4(x[0].x, x[1].x, x[2].x, x[3].x, l, ny);
                    acc[VEC > 1 ? 1 : 0].add4(x[0].y, x[1].y, x[2].y, x[3].y, l, ny);
                    acc[VEC > 2 ? 2 : 0].add4(x[0].z, x[1].z, x[2].z, x[3].z, l, ny);
                    acc[VEC > 3 ? 3 : 0].add4(x[0].w, x[1].w, x[2].w, x[3].w, l, ny);
                } else
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    long long ll = l + (long long)u * ny;
                    if (ok[u]) {
                        acc[0].add(x[u].x, ll);
                        acc[VEC > 1 ? 1 : 0].add(x[u].y, ll);
                        acc[VEC > 2 ? 2 : 0].add(x[u].z, ll);
                        acc[VEC > 3 ? 3 : 0].add(x[u].w, ll);
                    }
                }
            } else {
                float x[4];
                bool ok[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    long long ll = l + (long long)u * ny;
                    ok[u] = ll < l1;
                    if (ok[u]) x[u] = ld_stream1(base + ll * l_stride);
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    long long ll = l + (long long)u * ny;
                    if (ok[u]) acc[0].add(x[u], ll);
                }
            }
        }
    }
#pragma unroll
    for (int v = 0; v < VEC; ++v) acc[v].finish_thread();

    for (int stride = ny >> 1; stride >= 1; stride >>= 1) {
        if (ty >= stride && ty < 2 * stride) {
#pragma unroll
            for (int v = 0; v < VEC; ++v) sm[((ty - stride) * tx_n + tx) * VEC + v] = acc[v];
        }
        __syncthreads();
        if (ty < stride) {
#pragma unroll
            for (int v = 0; v < VEC; ++v) acc[v].merge(sm[(ty * tx_n + tx) * VEC + v]);
        }
        __syncthreads();
    }
    if (ty == 0 && active) {
#pragma unroll
        for (int v = 0; v < VEC; ++v) {
            if (ws) acc[v].store(TPB_CK(&ws[(o * S + s) * I + i0 + v]));
            else write_result(acc[v], e, (double)L, ov, oi, o * I + i0 + v);
        }
    }
}

template <class Acc>
__global__ void __launch_bounds__(256)
col_finalize_kernel(const Packed* __restrict__ ws, long long O, int S, long long I, double count,
                    Epilogue e, float* ov, long long* oi) {
    const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= O * I) return;
    const long long o = t / I, i = t - o * I;
    Acc acc;
    acc.load(TPB_CK(&ws[(o * S) * I + i]));
    for (int s = 1; s < S; ++s) {
        Acc b;
        b.load(TPB_CK(&ws[(o * S + s) * I + i]));
        acc.merge(b);
    }
    write_result(acc, e, count, ov, oi, t);
}

// ------------------------------------------------------------------ GENERIC ----------------
// One warp per output; addresses from a div/mod walk over the kept and the reduced dims.  Correct
// for every strided view (and for empty reductions: count = 0 leaves the start value).
template <class Acc>
__global__ void __launch_bounds__(256)
generic_kernel(const float* __restrict__ in, GenGeom g, Epilogue e, float* ov, long long* oi) {
    const int lane = threadIdx.x & 31;
    const long long o = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (o >= g.outs) return;
    long long off = 0, q = o;
    for (int d = g.nk - 1; d >= 0; --d) {
        long long c = q % g.ksize[d];
        q /= g.ksize[d];
        off += c * g.kstride[d];
    }
    Acc acc;
    acc.init();
    for (long long j = lane; j < g.count; j += 32) {
        long long roff = 0, jj = j;
        for (int d = g.nr - 1; d >= 0; --d) {
            long long c = jj % g.rsize[d];
            jj /= g.rsize[d];
            roff += c * g.rstride[d];
        }
        acc.add(ld_stream1(in + off + roff), j);
    }
    acc.finish_thread();
    warp_combine(acc);
    if (lane == 0) write_result(acc, e, (double)g.count, ov, oi, o);
}

// ------------------------------------------------------------------ planner ----------------
enum Family { FAM_SUM, FAM_MOM, FAM_MAX, FAM_MIN,
              // whole-op families without a sharded form
              FAM_PROD, FAM_NORM1, FAM_NORM2, FAM_ABSMAX, FAM_ABSMIN, FAM_ALL, FAM_ANY };
enum Strategy { ST_NONE, ST_ROW_WARP, ST_ROW_CTA, ST_ROW_SPLIT, ST_COL, ST_GENERIC };

struct Plan {
    Strategy st = ST_NONE;
    RowGeom row{};
    GenGeom gen{};
    // row
    int threads = 256, tps = 1, vec_ok = 0;
    int S = 1;
    long long chunk = 0;
    // col
    long long O = 1, o_stride = 0, L = 0, l_stride = 0, I = 0, lchunk = 0;
    int tiles = 1, tx_n = 1, vec = 1;
    long long outs = 0, count = 0;
    size_t ws_bytes = 0;
};

static int family_of(int op, Family* f) {
    switch (op) {
        case TPB200_OP_SUM: case TPB200_OP_MEAN: *f = FAM_SUM; return 0;
        case TPB200_OP_VAR: case TPB200_OP_STD: *f = FAM_MOM; return 0;
        case TPB200_OP_MAX: case TPB200_OP_ARGMAX: case TPB200_OP_MAX_ARGMAX: *f = FAM_MAX; return 0;
        case TPB200_OP_MIN: case TPB200_OP_ARGMIN: case TPB200_OP_MIN_ARGMIN: *f = FAM_MIN; return 0;
        case TPB200_OP_PROD: *f = FAM_PROD; return 0;
        case TPB200_OP_NORM1: *f = FAM_NORM1; return 0;
        case TPB200_OP_NORM2: *f = FAM_NORM2; return 0;
        case TPB200_OP_NORM_INF: *f = FAM_ABSMAX; return 0;
        case TPB200_OP_NORM_NEG_INF: *f = FAM_ABSMIN; return 0;
        case TPB200_OP_ALL: *f = FAM_ALL; return 0;
        case TPB200_OP_ANY: *f = FAM_ANY; return 0;
        default: return 1;
    }
}


constexpr long long kSplitBlock = 32768;   // elements per block of a split row: 512 threads x 4 loads of 16 bytes x 4 rounds

// CTAs per SM of a split reduction: as many as are resident at once (four of 512 threads; three for
// the variance, whose kernel needs 40 registers per thread), so that the whole launch is one wave.
static long long split_ctas_per_sm(Family fam) {
    int ev = 0;
    if (env_int("TPB200_SPLIT_PER_SM", &ev)) return std::max(1, ev);
    return fam == FAM_MOM ? 3 : 4;
}

struct Dim { long long size, stride; };

static void push_merged(std::vector<Dim>& v, Dim d) {
    if (!v.empty() && v.back().stride == d.stride * d.size) {
        v.back().size *= d.size;
        v.back().stride = d.stride;
    } else {
        v.push_back(d);
    }
}

// Override for experiments and tests: TPB200_FORCE_STRATEGY = warp | cta | split | col | generic
static Strategy forced_strategy() {
    const char* s = env_str("TPB200_FORCE_STRATEGY");
    if (!s) return ST_NONE;
    std::string v(s);
    if (v == "warp") return ST_ROW_WARP;
    if (v == "cta") return ST_ROW_CTA;
    if (v == "split") return ST_ROW_SPLIT;
    if (v == "col") return ST_COL;
    if (v == "generic") return ST_GENERIC;
    return ST_NONE;
}

static int make_plan(const void* in, int ndim, const int64_t* sizes, const int64_t* strides,
                     uint64_t mask, Family fam, Plan* pl) {
    if (ndim < 0 || ndim > TPB200_MAX_DIMS)
        return fail(TPB200_ERR_UNSUPPORTED, "tensors of rank %d are not supported (max %d)", ndim, TPB200_MAX_DIMS);
    if (ndim > 0 && (!sizes || !strides)) return fail(TPB200_ERR_INVALID, "sizes/strides must not be NULL");
    if (ndim < 64 && (mask >> ndim) != 0 && ndim > 0) return fail(TPB200_ERR_DIM_RANGE, "Dimension out of range");
    if (ndim == 0 && mask > 1) return fail(TPB200_ERR_DIM_RANGE, "Dimension out of range");
    const uint64_t all = ndim == 0 ? 0 : ((ndim == 64) ? ~0ull : ((1ull << ndim) - 1));
    if (mask == 0 || ndim == 0) mask = all;

    std::vector<Dim> kept, red;
    long long outs = 1, count = 1;
    for (int d = 0; d < ndim; ++d) {
        if (sizes[d] < 0) return fail(TPB200_ERR_INVALID, "negative size in dim %d", d);
        const bool r = (mask >> d) & 1;
        if (r) count *= sizes[d]; else outs *= sizes[d];
        if (sizes[d] == 1) continue;
        push_merged(r ? red : kept, Dim{sizes[d], strides[d]});
    }
    pl->outs = outs;
    pl->count = count;
    if (outs == 0) { pl->st = ST_NONE; return TPB200_OK; }

    const Strategy force = forced_strategy();
    const int sms = sm_count();
    const bool ptr16 = (((uintptr_t)in) & 15) == 0;

    auto use_generic = [&]() {
        GenGeom& g = pl->gen;
        g.nk = (int)kept.size();
        g.nr = (int)red.size();
        for (int i = 0; i < g.nk; ++i) { g.ksize[i] = kept[i].size; g.kstride[i] = kept[i].stride; }
        for (int i = 0; i < g.nr; ++i) { g.rsize[i] = red[i].size; g.rstride[i] = red[i].stride; }
        g.outs = outs;
        g.count = count;
        pl->st = ST_GENERIC;
        return TPB200_OK;
    };
    if (count == 0 || force == ST_GENERIC) return use_generic();
    if (red.empty()) red.push_back(Dim{1, 1});  // every reduced dim has size 1: rows of one element

    const bool row_ok = red.back().stride == 1 && red.size() <= 2 && kept.size() <= 2;
    const bool col_ok = red.size() == 1 && !kept.empty() && kept.back().stride == 1 && kept.size() <= 2;

    if (row_ok && force != ST_COL) {
        RowGeom& g = pl->row;
        g.rows = outs;
        g.seglen = red.back().size;
        g.nseg = red.size() == 2 ? red[0].size : 1;
        g.seg_stride = red.size() == 2 ? red[0].stride : 0;
        if (kept.size() == 2) { g.k1 = kept[1].size; g.ks0 = kept[0].stride; g.ks1 = kept[1].stride; }
        else if (kept.size() == 1) { g.k1 = 1; g.ks0 = kept[0].stride; g.ks1 = 0; }
        else { g.k1 = 1; g.ks0 = 0; g.ks1 = 0; }
        const long long L = g.nseg * g.seglen;
        pl->vec_ok = ptr16 && g.ks0 % 4 == 0 && g.ks1 % 4 == 0 && g.seg_stride % 4 == 0 && g.seglen % 4 == 0;

        // split: few rows, each long enough to feed many CTAs
        int S = 1;
        if (g.nseg == 1 && outs <= 0x3fffff) {
            long long want = std::max(1LL, (long long)sms * split_ctas_per_sm(fam) / outs);
            long long most = L / 16384;
            S = (int)std::max(1LL, std::min(std::min(want, most), 1LL << 20));
            // At least one row per SM and a launch of tens of microseconds: a CTA per row, one launch and
            // no partials.  Measured on [256,151936] over dim -1: 26.3 us (sum) / 26.8 us (max) against
            // 28.2 / 29.9 us with every row split in two (two launches for a 27 us stream).
            if (outs >= sms && outs * L * 4 <= (512LL << 20)) S = 1;
        }
        Strategy st;
        if (force == ST_ROW_SPLIT && g.nseg == 1 && outs <= 0x3fffff) { st = ST_ROW_SPLIT; S = std::max(S, 2); }
        else if (force == ST_ROW_WARP) st = ST_ROW_WARP;
        else if (force == ST_ROW_CTA) st = ST_ROW_CTA;
        else if (S >= 2) st = ST_ROW_SPLIT;
        else if (g.nseg == 1 && (L <= 1024 || (L <= 8192 && outs >= 8LL * sms))) st = ST_ROW_WARP;
        // (rows of up to 32 KB with at least one warp-row per warp slot of the GPU: a warp per row
        //  needs no shared-memory combine and a fraction of the instructions of a CTA per row)
        else st = ST_ROW_CTA;

        pl->st = st;
        if (st == ST_ROW_SPLIT) {
            pl->chunk = kSplitBlock;                       // block length of the interleaved walk
            pl->S = (int)std::max(1LL, std::min<long long>(S, ceil_div(L, pl->chunk)));
            pl->threads = 512;
            pl->ws_bytes = (size_t)outs * pl->S * sizeof(Packed);
        } else if (st == ST_ROW_CTA) {
            pl->threads = L <= 2048 ? 128 : (L <= 16384 ? 256 : 512);
            pl->tps = g.nseg == 1 ? pl->threads : std::min(pl->threads, pow2_ceil(std::max(1LL, g.seglen / 4)));
        }
        return TPB200_OK;
    }
    if (col_ok) {
        pl->st = ST_COL;
        pl->I = kept.back().size;
        pl->L = red[0].size;
        pl->l_stride = red[0].stride;
        if (kept.size() == 2) { pl->O = kept[0].size; pl->o_stride = kept[0].stride; }
        else { pl->O = 1; pl->o_stride = 0; }
        pl->vec = (ptr16 && pl->I % 4 == 0 && pl->o_stride % 4 == 0 && pl->l_stride % 4 == 0) ? 4 : 1;
        pl->tx_n = std::min(32, pow2_ceil(ceil_div(pl->I, pl->vec)));
        pl->tiles = (int)ceil_div(pl->I, (long long)pl->tx_n * pl->vec);
        const int ny = 256 / pl->tx_n;
        long long ctas = pl->O * pl->tiles;
        // one wave -- as many slices as keep all CTAs resident at once (4 CTAs of 256 threads per SM);
        // measured on [64,4096,512] over dim 1: sum 2 slices (512 CTAs) 82 us, 5 slices (1280 CTAs)
        // 96 us; variance 2 slices 91 us, 5 slices 128 us
        long long want = std::max(1LL, ((long long)sms * 4) / std::max(1LL, ctas));
        long long most = std::max(1LL, pl->L / ((long long)ny * 8));
        int S = (int)std::max(1LL, std::min(std::min(want, most), 65535LL));
        int fs = 0;
        if (env_int("TPB200_COL_SPLITS", &fs)) S = (int)std::max(1LL, std::min<long long>(fs, most));
        pl->lchunk = ceil_div(pl->L, S);
        pl->S = (int)ceil_div(pl->L, pl->lchunk);
        if (pl->S > 1) pl->ws_bytes = (size_t)pl->O * pl->S * pl->I * sizeof(Packed);
        if (pl->O * pl->tiles > 0x7fffffffLL) return use_generic();
        return TPB200_OK;
    }
    return use_generic();
}

template <class Acc>
static int launch_plan(const Plan& pl, const float* in, Epilogue e, float* ov, long long* oi,
                       void* ws, cudaStream_t st) {
    switch (pl.st) {
        case ST_NONE:
            return TPB200_OK;
        case ST_ROW_WARP: {
            // rows per CTA: eight, or four where that spreads one wave of CTAs more evenly over the
            // SMs (4096 rows: 512 CTAs are 3.46 per SM, i.e. 4 on some and 3 on others; 1024 CTAs
            // are 6.92 per SM)
            int wpc = 8;
            {
                const double sms = (double)sm_count();
                const double a8 = (double)ceil_div(pl.row.rows, 8) / sms, a4 = (double)ceil_div(pl.row.rows, 4) / sms;
                if (a4 <= 10.0 && std::ceil(a4) / a4 < std::ceil(a8) / a8 - 0.02) wpc = 4;
            }
            if (pl.row.nseg == 1 && pl.row.seglen <= 256 && pl.row.rows >= 4096) {
                const int G = pl.row.seglen <= 64 ? 4 : (pl.row.seglen <= 128 ? 8 : 16);
                const long long warps = ceil_div(pl.row.rows, 32 / G);
                const dim3 gg((unsigned)ceil_div(warps, 8));
                if (G == 4)      TPB_LAUNCH("row_group_kernel", (row_group_kernel<Acc, 4>), gg, 256, 0, st, in, pl.row, e, ov, oi);
                else if (G == 8) TPB_LAUNCH("row_group_kernel", (row_group_kernel<Acc, 8>), gg, 256, 0, st, in, pl.row, e, ov, oi);
                else             TPB_LAUNCH("row_group_kernel", (row_group_kernel<Acc, 16>), gg, 256, 0, st, in, pl.row, e, ov, oi);
                return TPB200_OK;
            }
            unsigned grid = (unsigned)ceil_div(pl.row.rows, wpc);
            if (pl.row.seglen >= 2048) TPB_LAUNCH("row_warp_long_kernel", row_warp_long_kernel<Acc>, dim3(grid), wpc * 32, 0, st, in, pl.row, e, ov, oi);
            else                       TPB_LAUNCH("row_warp_kernel", row_warp_kernel<Acc>, dim3(grid), wpc * 32, 0, st, in, pl.row, e, ov, oi);
            return TPB200_OK;
        }
        case ST_ROW_CTA: {
            if (pl.row.rows > 0x7fffffffLL) return fail(TPB200_ERR_UNSUPPORTED, "too many rows for one launch");
            TPB_LAUNCH("row_cta_kernel", row_cta_kernel<Acc>, dim3((unsigned)pl.row.rows), pl.threads, 0, st, in, pl.row, pl.tps, pl.vec_ok, e, ov, oi);
            return TPB200_OK;
        }
        case ST_ROW_SPLIT: {
            if (pl.row.rows * pl.S > 0x7fffffffLL) return fail(TPB200_ERR_UNSUPPORTED, "too many rows for one launch");
            dim3 grid((unsigned)(pl.S * pl.row.rows));
            TPB_LAUNCH("row_split_kernel", row_split_kernel<Acc>, grid, pl.threads, 0, st, in, pl.row, pl.chunk, pl.S, (Packed*)ws);
            unsigned fg = (unsigned)ceil_div(pl.row.rows, 4);
            TPB_LAUNCH("finalize_kernel", finalize_kernel<Acc>, dim3(fg), 128, 0, st, (const Packed*)ws, pl.row.rows, pl.S, (double)pl.count, e, ov, oi,
                       (Packed*)nullptr, 0LL);
            return TPB200_OK;
        }
        case ST_COL: {
            const int ny = 256 / pl.tx_n;
            dim3 grid((unsigned)(pl.O * pl.tiles), (unsigned)pl.S);
            Packed* w = pl.S > 1 ? (Packed*)ws : nullptr;
            if (pl.vec == 4) {
                size_t sm = (size_t)std::max(1, ny / 2) * pl.tx_n * 4 * sizeof(Acc);
                TPB_LAUNCH("col_kernel", (col_kernel<Acc, 4>), grid, 256, sm, st, in, pl.o_stride, pl.L, pl.l_stride, pl.I, pl.tiles, pl.tx_n, pl.lchunk, w, e, ov, oi);
            } else {
                size_t sm = (size_t)std::max(1, ny / 2) * pl.tx_n * sizeof(Acc);
                TPB_LAUNCH("col_kernel", (col_kernel<Acc, 1>), grid, 256, sm, st, in, pl.o_stride, pl.L, pl.l_stride, pl.I, pl.tiles, pl.tx_n, pl.lchunk, w, e, ov, oi);
            }
            if (pl.S > 1) {
                unsigned fg = (unsigned)ceil_div(pl.O * pl.I, 256);
                TPB_LAUNCH("col_finalize_kernel", col_finalize_kernel<Acc>, dim3(fg), 256, 0, st, (const Packed*)ws, pl.O, pl.S, pl.I, (double)pl.count, e, ov, oi);
            }
            return TPB200_OK;
        }
        case ST_GENERIC: {
            unsigned grid = (unsigned)ceil_div(pl.gen.outs, 8);
            TPB_LAUNCH("generic_kernel", generic_kernel<Acc>, dim3(grid), 256, 0, st, in, pl.gen, e, ov, oi);
            return TPB200_OK;
        }
    }
    return fail(TPB200_ERR_INVALID, "internal: no strategy");
}

static int check_ws(const Plan& pl, void* ws, size_t ws_bytes) {
    if (pl.ws_bytes == 0) return TPB200_OK;
    if (!ws || ws_bytes < pl.ws_bytes)
        return fail(TPB200_ERR_WORKSPACE, "workspace of %zu bytes required, %zu given", pl.ws_bytes, ws ? ws_bytes : (size_t)0);
    if (((uintptr_t)ws) & 7) return fail(TPB200_ERR_WORKSPACE, "workspace must be 8-byte aligned");
    return TPB200_OK;
}

}  // namespace tpb

using namespace tpb;

extern "C" size_t tpb200_reduce_workspace_bytes(int op, int dtype, int ndim, const int64_t* sizes,
                                                const int64_t* strides, uint64_t reduce_mask) {
    Family fam;
    if (dtype != TPB200_F32 || family_of(op, &fam)) return 0;
    Plan pl;
    // alignment of the data pointer does not change the workspace size
    if (make_plan((const void*)16, ndim, sizes, strides, reduce_mask, fam, &pl) != TPB200_OK) return 0;
    return pl.ws_bytes;
}

extern "C" int tpb200_reduce(int op, const void* in, int dtype, int ndim, const int64_t* sizes,
                             const int64_t* strides, uint64_t reduce_mask, int index_dim,
                             int64_t correction, void* out_val, int64_t* out_idx, void* workspace,
                             size_t workspace_bytes, void* stream) {
    Family fam;
    if (family_of(op, &fam)) return fail(TPB200_ERR_INVALID, "unknown reduction operator %d", op);
    if (dtype != TPB200_F32) return fail(TPB200_ERR_UNSUPPORTED, "only float32 input is supported (dtype code %d)", dtype);
    const bool wants_val = !(op == TPB200_OP_ARGMAX || op == TPB200_OP_ARGMIN);
    const bool wants_idx = op == TPB200_OP_ARGMAX || op == TPB200_OP_ARGMIN || op == TPB200_OP_MAX_ARGMAX || op == TPB200_OP_MIN_ARGMIN;
    Plan pl;
    int rc = make_plan(in, ndim, sizes, strides, reduce_mask, fam, &pl);
    if (rc) return rc;
    if (wants_idx) {
        const uint64_t all = ndim == 0 ? 0 : ((1ull << ndim) - 1);
        if (index_dim < 0) {
            if (!(reduce_mask == 0 || reduce_mask == all))
                return fail(TPB200_ERR_INVALID, "a flat index needs every dim reduced");
        } else {
            if (index_dim >= ndim) return fail(TPB200_ERR_DIM_RANGE, "Dimension out of range");
            if (reduce_mask != (1ull << index_dim))
                return fail(TPB200_ERR_INVALID, "index_dim must be the one reduced dim");
        }
    }
    if (pl.outs == 0) return TPB200_OK;
    if (wants_val && (fam == FAM_MAX || fam == FAM_MIN || fam == FAM_ABSMAX || fam == FAM_ABSMIN) && pl.count == 0 && reduce_mask == 0) {
        // the overload without a dim argument on an empty tensor (ReductionKernels.cpp:240, :326);
        // with an explicit dim list the reference fills the output with the start value instead
        return fail(TPB200_ERR_EMPTY, "%s(): Expected reduction dim to be non-empty", (fam == FAM_MAX || fam == FAM_ABSMAX) ? "max" : "min");
    }
    if (!in && pl.count > 0) return fail(TPB200_ERR_INVALID, "input pointer is NULL");
    if (wants_val && !out_val) return fail(TPB200_ERR_INVALID, "out_val is NULL");
    if (wants_idx && !out_idx) return fail(TPB200_ERR_INVALID, "out_idx is NULL");
    rc = check_ws(pl, workspace, workspace_bytes);
    if (rc) return rc;

    Epilogue e{op, (long long)correction};
    float* ov = wants_val ? (float*)out_val : nullptr;
    long long* oi = wants_idx ? (long long*)out_idx : nullptr;
    cudaStream_t st = (cudaStream_t)stream;
    const float* x = (const float*)in;
    TPB_CHECK_RANGES(st, view_range(in, ndim, sizes, strides, 4),
                     HostRange{ov, (size_t)pl.outs * ((fam == FAM_ALL || fam == FAM_ANY) ? 1 : 4)},
                     HostRange{oi, (size_t)pl.outs * 8}, HostRange{workspace, pl.ws_bytes});
    switch (fam) {
        case FAM_SUM: return launch_plan<SumAcc>(pl, x, e, ov, oi, workspace, st);
        case FAM_MOM: return launch_plan<MomAcc>(pl, x, e, ov, oi, workspace, st);
        case FAM_MAX: return launch_plan<ExtAcc<true>>(pl, x, e, ov, oi, workspace, st);
        case FAM_MIN: return launch_plan<ExtAcc<false>>(pl, x, e, ov, oi, workspace, st);
        case FAM_PROD: return launch_plan<ProdAcc>(pl, x, e, ov, oi, workspace, st);
        case FAM_NORM1: return launch_plan<PowSumAcc<0>>(pl, x, e, ov, oi, workspace, st);
        case FAM_NORM2: return launch_plan<PowSumAcc<1>>(pl, x, e, ov, oi, workspace, st);
        case FAM_ABSMAX: return launch_plan<ExtAcc<true, true>>(pl, x, e, ov, oi, workspace, st);
        case FAM_ABSMIN: return launch_plan<ExtAcc<false, true>>(pl, x, e, ov, oi, workspace, st);
        case FAM_ALL: return launch_plan<BoolAcc<true>>(pl, x, e, ov, oi, workspace, st);
        case FAM_ANY: return launch_plan<BoolAcc<false>>(pl, x, e, ov, oi, workspace, st);
    }
    return fail(TPB200_ERR_INVALID, "internal: bad family");
}

// ---------------------------------------------------------------- sharded whole tensor ------
namespace tpb {

static void flat_plan(const void* in, int64_t n, Family fam, Plan* pl) {
    const int sms = sm_count();
    RowGeom& g = pl->row;
    g.rows = 1; g.k1 = 1; g.ks0 = 0; g.ks1 = 0; g.nseg = 1; g.seglen = n; g.seg_stride = 0;
    long long S = std::max(1LL, std::min((long long)sms * split_ctas_per_sm(fam), (long long)(n / 16384)));
    pl->chunk = kSplitBlock;
    pl->S = (int)std::max(1LL, std::min(S, ceil_div(std::max<long long>(n, 1), pl->chunk)));
    pl->threads = 512;
    pl->outs = 1;
    pl->count = n;
    pl->ws_bytes = (size_t)std::max(1LL, std::min((long long)sms * 16, (long long)(n / 16384) + 1)) * sizeof(Packed);
    pl->st = ST_ROW_SPLIT;
    (void)in;
}

template <class Acc>
static int launch_partial(const Plan& pl, const float* in, long long offset, Packed* out, void* ws,
                          cudaStream_t st) {
    TPB_LAUNCH("row_split_kernel", row_split_kernel<Acc>, dim3((unsigned)pl.S), pl.threads, 0, st, in, pl.row, pl.chunk, pl.S, (Packed*)ws);
    Epilogue e{0, 0};
    TPB_LAUNCH("finalize_kernel", finalize_kernel<Acc>, dim3(1), 32, 0, st, (const Packed*)ws, 1LL, pl.S, (double)pl.count, e, (float*)nullptr,
               (long long*)nullptr, out, offset);
    return TPB200_OK;
}

template <class Acc>
static int launch_combine(const Packed* parts, int n, double count, Epilogue e, float* ov,
                          long long* oi, cudaStream_t st) {
    TPB_LAUNCH("finalize_kernel", finalize_kernel<Acc>, dim3(1), 32, 0, st, parts, 1LL, n, count, e, ov, oi, (Packed*)nullptr, 0LL);
    return TPB200_OK;
}

}  // namespace tpb

extern "C" size_t tpb200_reduce_partial_workspace_bytes(int family, int dtype, int64_t n) {
    (void)family;
    if (dtype != TPB200_F32 || n < 0) return 0;
    Plan pl;
    flat_plan(nullptr, n, FAM_SUM, &pl);   // the size covers every family
    return pl.ws_bytes;
}

extern "C" int tpb200_reduce_partial(int family, const void* in, int dtype, int64_t n,
                                     int64_t global_offset, void* partial_out, void* workspace,
                                     size_t workspace_bytes, void* stream) {
    Family fam;
    if (family_of(family, &fam)) return fail(TPB200_ERR_INVALID, "unknown reduction family %d", family);
    if (fam > FAM_MIN) return fail(TPB200_ERR_UNSUPPORTED, "operator %d has no sharded form", family);
    if (dtype != TPB200_F32) return fail(TPB200_ERR_UNSUPPORTED, "only float32 input is supported (dtype code %d)", dtype);
    if (n < 0) return fail(TPB200_ERR_INVALID, "negative element count");
    if (!partial_out) return fail(TPB200_ERR_INVALID, "partial_out is NULL");
    if (n > 0 && !in) return fail(TPB200_ERR_INVALID, "input pointer is NULL");
    if (((uintptr_t)partial_out) & 7) return fail(TPB200_ERR_INVALID, "partial_out must be 8-byte aligned");
    Plan pl;
    flat_plan(in, n, fam, &pl);
    int rc = check_ws(pl, workspace, workspace_bytes);
    if (rc) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    const float* x = (const float*)in;
    Packed* out = (Packed*)partial_out;
    TPB_CHECK_RANGES(st, HostRange{in, (size_t)n * 4}, HostRange{partial_out, sizeof(Packed)}, HostRange{workspace, pl.ws_bytes});
    switch (fam) {
        case FAM_SUM: return launch_partial<SumAcc>(pl, x, global_offset, out, workspace, st);
        case FAM_MOM: return launch_partial<MomAcc>(pl, x, global_offset, out, workspace, st);
        case FAM_MAX: return launch_partial<ExtAcc<true>>(pl, x, global_offset, out, workspace, st);
        case FAM_MIN: return launch_partial<ExtAcc<false>>(pl, x, global_offset, out, workspace, st);
    }
    return fail(TPB200_ERR_INVALID, "internal: bad family");
}

extern "C" int tpb200_reduce_combine(int op, const void* partials, int n_parts, int64_t total_count,
                                     int64_t correction, void* out_val, int64_t* out_idx, void* stream) {
    Family fam;
    if (family_of(op, &fam)) return fail(TPB200_ERR_INVALID, "unknown reduction operator %d", op);
    if (fam > FAM_MIN) return fail(TPB200_ERR_UNSUPPORTED, "operator %d has no sharded form", op);
    if (n_parts < 1 || !partials) return fail(TPB200_ERR_INVALID, "need at least one partial record");
    const bool wants_val = !(op == TPB200_OP_ARGMAX || op == TPB200_OP_ARGMIN);
    const bool wants_idx = op == TPB200_OP_ARGMAX || op == TPB200_OP_ARGMIN || op == TPB200_OP_MAX_ARGMAX || op == TPB200_OP_MIN_ARGMIN;
    if (wants_val && !out_val) return fail(TPB200_ERR_INVALID, "out_val is NULL");
    if (wants_idx && !out_idx) return fail(TPB200_ERR_INVALID, "out_idx is NULL");
    Epilogue e{op, (long long)correction};
    float* ov = wants_val ? (float*)out_val : nullptr;
    long long* oi = wants_idx ? (long long*)out_idx : nullptr;
    cudaStream_t st = (cudaStream_t)stream;
    const Packed* p = (const Packed*)partials;
    const double cnt = (double)total_count;
    TPB_CHECK_RANGES(st, HostRange{partials, (size_t)n_parts * sizeof(Packed)}, HostRange{ov, 4}, HostRange{oi, 8});
    switch (fam) {
        case FAM_SUM: return launch_combine<SumAcc>(p, n_parts, cnt, e, ov, oi, st);
        case FAM_MOM: return launch_combine<MomAcc>(p, n_parts, cnt, e, ov, oi, st);
        case FAM_MAX: return launch_combine<ExtAcc<true>>(p, n_parts, cnt, e, ov, oi, st);
        case FAM_MIN: return launch_combine<ExtAcc<false>>(p, n_parts, cnt, e, ov, oi, st);
    }
    return fail(TPB200_ERR_INVALID, "internal: bad family");
}

// ---------------------------------------------------------------- no-allocation variant ------
// Whole-tensor reduction for callers that may not allocate device memory and have no scratch
// buffer of their own to lend: a host that has handed every byte of the device to its own memory
// pool, or a latency-critical loop that cannot afford the implicit device-wide synchronisation of
// cudaMalloc / cudaFree.  It is the split-row reduction above (row_split_kernel + finalize_kernel)
// with the packed partials kept in a fixed array inside this module instead of a caller workspace.
//
// The array lives in every GPU that loads the library until the process exits (128 KiB each).
// In host code its name is only a stand-in; the device address is fetched once per device with
// cudaGetSymbolAddress (with that device current) and handed to the kernels as a plain pointer.
namespace tpb {

static __device__ __align__(256) unsigned char g_noalloc_scratch[TPB200_NOALLOC_SCRATCH_BYTES];

// Device address of the array on the current device (looked up on the first call per device).
static int noalloc_scratch_address(void** out) {
    static std::mutex mu;
    static void* cached[64];
    int dev = 0;
    TPB_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(TPB200_ERR_UNSUPPORTED, "device ordinal %d is not supported", dev);
    std::lock_guard<std::mutex> lk(mu);
    if (!cached[dev]) {
        void* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress((void**)&p, g_noalloc_scratch);
        if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(g_noalloc_scratch)");
        if (!p) return fail(TPB200_ERR_CUDA, "CUDA Error: no device address for the scratch array");
        cached[dev] = p;
    }
    *out = cached[dev];
    return TPB200_OK;
}

}  // namespace tpb

extern "C" int tpb200_reduce_all_noalloc(int op, const void* in, int dtype, int64_t n, int64_t correction,
                                         void* out_val, int64_t* out_idx, void* stream) {
    Family fam;
    if (family_of(op, &fam)) return fail(TPB200_ERR_INVALID, "unknown reduction operator %d", op);
    if (fam > FAM_MIN) return fail(TPB200_ERR_UNSUPPORTED, "operator %d has no sharded form", op);
    if (dtype != TPB200_F32) return fail(TPB200_ERR_UNSUPPORTED, "only float32 input is supported (dtype code %d)", dtype);
    if (n < 0) return fail(TPB200_ERR_INVALID, "negative element count");
    if ((uint64_t)n > (uint64_t)TPB200_NOALLOC_MAX_ELEMENTS)
        return fail(TPB200_ERR_UNSUPPORTED, "tpb200_reduce_all_noalloc handles at most %llu elements, %lld given",
                    (unsigned long long)TPB200_NOALLOC_MAX_ELEMENTS, (long long)n);
    const bool wants_val = !(op == TPB200_OP_ARGMAX || op == TPB200_OP_ARGMIN);
    const bool wants_idx = op == TPB200_OP_ARGMAX || op == TPB200_OP_ARGMIN || op == TPB200_OP_MAX_ARGMAX || op == TPB200_OP_MIN_ARGMIN;
    if (wants_val && (fam == FAM_MAX || fam == FAM_MIN) && n == 0)
        return fail(TPB200_ERR_EMPTY, "%s(): Expected reduction dim to be non-empty", fam == FAM_MAX ? "max" : "min");
    if (n > 0 && !in) return fail(TPB200_ERR_INVALID, "input pointer is NULL");
    if (wants_val && !out_val) return fail(TPB200_ERR_INVALID, "out_val is NULL");
    if (wants_idx && !out_idx) return fail(TPB200_ERR_INVALID, "out_idx is NULL");

    // the very plan tpb200_reduce makes for a contiguous 1-D tensor with every dim reduced, so the
    // two entry points run the same kernels in the same geometry and agree bit for bit
    Plan pl;
    const int64_t sizes1[1] = {n}, strides1[1] = {1};
    int prc = make_plan(in, 1, sizes1, strides1, 0, fam, &pl);
    if (prc) return prc;
    if (pl.ws_bytes > (size_t)TPB200_NOALLOC_SCRATCH_BYTES)
        return fail(TPB200_ERR_UNSUPPORTED, "this device needs %zu bytes of scratch, the built-in array holds %d",
                    pl.ws_bytes, (int)TPB200_NOALLOC_SCRATCH_BYTES);
    void* scratch = nullptr;
    int rc = noalloc_scratch_address(&scratch);
    if (rc) return rc;

    // Short inputs need no scratch at all (one warp or one CTA reduces them).  Pass 1 overwrites every record that pass 2 reads, so nothing left by an earlier call is used
    // and nothing has to be cleared.
    Epilogue e{op, (long long)correction};
    float* ov = wants_val ? (float*)out_val : nullptr;
    long long* oi = wants_idx ? (long long*)out_idx : nullptr;
    cudaStream_t st = (cudaStream_t)stream;
    const float* x = (const float*)in;
    TPB_CHECK_RANGES(st, HostRange{in, (size_t)n * 4}, HostRange{ov, 4}, HostRange{oi, 8}, HostRange{scratch, pl.ws_bytes});
    switch (fam) {
        case FAM_SUM: return launch_plan<SumAcc>(pl, x, e, ov, oi, scratch, st);
        case FAM_MOM: return launch_plan<MomAcc>(pl, x, e, ov, oi, scratch, st);
        case FAM_MAX: return launch_plan<ExtAcc<true>>(pl, x, e, ov, oi, scratch, st);
        case FAM_MIN: return launch_plan<ExtAcc<false>>(pl, x, e, ov, oi, scratch, st);
    }
    return fail(TPB200_ERR_INVALID, "internal: bad family");
}

// ---------------------------------------------------------------- fused partial + exchange ----
// Whole-tensor reduction of a flat tensor sharded over `world` GPUs without a library collective:
// row_split_kernel reduces the slices of this GPU's partition; finalize_exchange_kernel (one warp)
// merges them, writes this rank's 40-byte record straight into the exchange buffer of EVERY rank
// (plain peer-to-peer stores over NVLink; no multicast, no multimem), raises a per-rank epoch flag
// with release semantics at system scope, waits -- bounded -- until the flags of all ranks show the
// same epoch, and merges the `world` records in rank order.  Every rank computes the identical
// result.  Replaces finalize_kernel -> all-gather -> finalize_kernel of the unfused path by one
// kernel.  (Folding the exchange into the tail of row_split_kernel itself was measured too: the
// extra code cost the extremum variant 14% of its streaming rate, so the streaming kernel stays as
// it is and the exchange lives in the one-warp kernel that follows it.)
//
// Exchange buffer (one per rank, peer-mapped, zero-filled once before the first call):
//   Packed slots[2][kMaxPeers]   records of epoch parity 0 / 1 (a rank can run at most one call
//                                ahead of another: it needs the other's flag of its own epoch)
//   unsigned flags[kMaxPeers]    flags[j] = last epoch whose record rank j has delivered here
//   unsigned epoch, ticket       local call counter (ticket is unused padding)
// Every wait is bounded (tpb200_set_exchange_wait_polls; about half a second by default): a rank
// whose peers do not arrive in that time writes NaN / -1 to its outputs -- a timed-out call must not
// pass for a result: the output buffers may still hold the previous call's answer -- and sets the
// status word to kErrExchange.
namespace tpb {

constexpr int kMaxPeers = 16;
constexpr int kErrExchange = 5;
constexpr int kExchangePollsDefault = 1 << 22;   // polls of 100 ns and more each
constexpr int kExchangePollsMax = 1 << 25;       // a few seconds
static std::atomic<int> g_exchange_polls{kExchangePollsDefault};

struct ExchangeBuf {
    Packed slots[2][kMaxPeers];
    unsigned flags[kMaxPeers];
    unsigned epoch;
    unsigned ticket;
    unsigned pad[14];
};
struct PeerPtrs { ExchangeBuf* p[kMaxPeers]; };

__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// One warp: this rank's record from its S partials (fixed order), exchange, rank-ordered merge.
template <class Acc>
__global__ void __launch_bounds__(32)
finalize_exchange_kernel(const Packed* __restrict__ ws, int S, long long idx_offset, int rank, int world,
                         PeerPtrs peers, double total_count, Epilogue e, float* ov, long long* oi, int* status,
                         int max_polls) {
    const int lane = threadIdx.x & 31;
    if (lane == 0) TPB_RED_STAMP(2);
    ExchangeBuf* mine = peers.p[rank];
    Acc r;
    r.init();
    r.finish_thread();
    merge_partials(r, ws, S, lane);
    warp_combine(r);
    // Lane j talks to rank j: it stores this rank's record into rank j's buffer and then the flag with
    // release semantics (which orders that lane's record stores before the flag, all the way to the
    // peer), waits for rank j's flag and takes rank j's record.  All ranks are served at once: one lane
    // doing the eight stores, a system-wide fence and eight release stores in turn took 13-17 us of an
    // 8-GPU step; the flags and records of the peers cross NVLink in parallel this way.
    __shared__ Packed rec_sh;
    if (lane == 0) {
        TPB_RED_STAMP(3);
        r.store(&rec_sh);
        if (rec_sh.i0 != kNoIndex) rec_sh.i0 += idx_offset;
    }
    unsigned ep = lane == 0 ? *TPB_CK(&mine->epoch) + 1u : 0u;
    ep = __shfl_sync(kFull, ep, 0);
    __syncwarp();
    const int par = (int)(ep & 1u);
    bool ok = true;
    if (lane < world) {
        *TPB_CK(&peers.p[lane]->slots[par][rank]) = rec_sh;                 // peer-to-peer stores
        st_release_sys(TPB_CK(&peers.p[lane]->flags[rank]), ep);
    }
    __syncwarp();
    if (lane == 0) TPB_RED_STAMP(4);
    // the merge of the ranks' records: lane j holds rank j's, then the warp's fixed tree -- the order
    // of finalize_kernel over the same records, so both exchange paths give the same bits
    Acc all;
    all.init();
    all.finish_thread();
    if (lane < world) {
        // bounded wait for rank `lane`'s record of this epoch
        int spin = 0;
        while ((int)(ld_acquire_sys(TPB_CK(&mine->flags[lane])) - ep) < 0) {
            if (++spin > max_polls) { ok = false; break; }
            __nanosleep(100);
        }
        if (ok) {
            Acc o;
            o.load(TPB_CK(&mine->slots[par][lane]));
            all.merge(o);
        }
    }
    ok = __all_sync(kFull, ok);
    if (lane == 0) TPB_RED_STAMP(5);
    warp_combine(all);
    if (lane == 0) {
        *TPB_CK(&mine->epoch) = ep;
        if (!ok) {
            if (status) atomicMax(status, kErrExchange);
            if (ov) *TPB_CK(&ov[0]) = NAN;
            if (oi) *TPB_CK(&oi[0]) = -1;
        } else {
            write_result(all, e, total_count, ov, oi, 0);
        }
        TPB_RED_STAMP(6);
    }
}

}  // namespace tpb

#ifdef TPB200_TRACE
// Reads the seven stamps (nanoseconds of this GPU's %globaltimer) and re-arms them: slot 0 to the largest
// value (it is a minimum), the others to 0.
extern "C" int tpb200_debug_reduce_trace(unsigned long long* host, int n) {
    if (n > 8) n = 8;
    cudaError_t e = cudaMemcpyFromSymbol(host, tpb::g_red_trace, sizeof(unsigned long long) * n);
    if (e != cudaSuccess) return (int)e;
    unsigned long long init[8] = {~0ull, 0, 0, 0, 0, 0, 0, 0};
    return (int)cudaMemcpyToSymbol(tpb::g_red_trace, init, sizeof(init));
}
#endif

extern "C" size_t tpb200_exchange_buffer_bytes(void) { return sizeof(tpb::ExchangeBuf); }

extern "C" int tpb200_set_exchange_wait_polls(int polls) {
    if (polls < 1 || polls > tpb::kExchangePollsMax)
        return fail(TPB200_ERR_INVALID, "the exchange wait takes 1..%d polls, %d given", tpb::kExchangePollsMax, polls);
    tpb::g_exchange_polls.store(polls, std::memory_order_relaxed);
    return TPB200_OK;
}

extern "C" int tpb200_reduce_fused_exchange(int op, const void* in, int dtype, int64_t n, int64_t global_offset,
                                            int64_t total_count, int64_t correction, int rank, int world,
                                            void* const* peer_buffers, void* out_val, int64_t* out_idx,
                                            void* workspace, size_t workspace_bytes, void* stream) {
    Family fam;
    if (family_of(op, &fam)) return fail(TPB200_ERR_INVALID, "unknown reduction operator %d", op);
    if (fam > FAM_MIN) return fail(TPB200_ERR_UNSUPPORTED, "operator %d has no sharded form", op);
    if (dtype != TPB200_F32) return fail(TPB200_ERR_UNSUPPORTED, "only float32 input is supported (dtype code %d)", dtype);
    if (n < 0 || total_count < n) return fail(TPB200_ERR_INVALID, "bad element counts");
    if (world < 1 || world > kMaxPeers) return fail(TPB200_ERR_UNSUPPORTED, "1..%d ranks are supported, %d given", kMaxPeers, world);
    if (rank < 0 || rank >= world) return fail(TPB200_ERR_INVALID, "rank %d outside 0..%d", rank, world - 1);
    if (!peer_buffers) return fail(TPB200_ERR_INVALID, "peer_buffers is NULL");
    PeerPtrs peers{};
    for (int j = 0; j < world; ++j) {
        if (!peer_buffers[j] || (((uintptr_t)peer_buffers[j]) & 7)) return fail(TPB200_ERR_INVALID, "exchange buffer of rank %d is NULL or misaligned", j);
        peers.p[j] = (ExchangeBuf*)peer_buffers[j];
    }
    const bool wants_val = !(op == TPB200_OP_ARGMAX || op == TPB200_OP_ARGMIN);
    const bool wants_idx = op == TPB200_OP_ARGMAX || op == TPB200_OP_ARGMIN || op == TPB200_OP_MAX_ARGMAX || op == TPB200_OP_MIN_ARGMIN;
    if (wants_val && !out_val) return fail(TPB200_ERR_INVALID, "out_val is NULL");
    if (wants_idx && !out_idx) return fail(TPB200_ERR_INVALID, "out_idx is NULL");
    if (n > 0 && !in) return fail(TPB200_ERR_INVALID, "input pointer is NULL");
    Plan pl;
    flat_plan(in, n, fam, &pl);
    int rc = check_ws(pl, workspace, workspace_bytes);
    if (rc) return rc;
    Epilogue e{op, (long long)correction};
    float* ov = wants_val ? (float*)out_val : nullptr;
    long long* oi = wants_idx ? (long long*)out_idx : nullptr;
    cudaStream_t st = (cudaStream_t)stream;
    const float* x = (const float*)in;
    int* status = device_status_word();
    const double tc = (double)total_count;
    const int max_polls = g_exchange_polls.load(std::memory_order_relaxed);
#ifdef TPB200_CHECKED
    {
        HostRange rr[4 + kMaxPeers] = {HostRange{in, (size_t)n * 4}, HostRange{ov, 4}, HostRange{oi, 8}, HostRange{workspace, pl.ws_bytes}};
        for (int j = 0; j < world; ++j) rr[4 + j] = HostRange{peer_buffers[j], sizeof(ExchangeBuf)};
        const int crc = check_register(st, rr, 4 + world);
        if (crc) return crc;
    }
#endif
#define TPB_LAUNCH_X(ACC)                                                                                    \
    do {                                                                                                     \
        TPB_LAUNCH("row_split_kernel", row_split_kernel<ACC>, dim3((unsigned)pl.S), pl.threads, 0, st, x, pl.row, pl.chunk, pl.S, (Packed*)workspace); \
        TPB_LAUNCH("finalize_exchange_kernel", finalize_exchange_kernel<ACC>, dim3(1), 32, 0, st, (const Packed*)workspace, pl.S, \
                   (long long)global_offset, rank, world, peers, tc, e, ov, oi, status, max_polls);          \
    } while (0)
    switch (fam) {
        case FAM_SUM: TPB_LAUNCH_X(SumAcc); break;
        case FAM_MOM: TPB_LAUNCH_X(MomAcc); break;
        case FAM_MAX: TPB_LAUNCH_X(ExtAcc<true>); break;
        case FAM_MIN: TPB_LAUNCH_X(ExtAcc<false>); break;
    }
#undef TPB_LAUNCH_X
    return TPB200_OK;
}
