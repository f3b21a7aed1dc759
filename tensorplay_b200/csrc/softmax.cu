// softmax / log_softmax along one dim for float32 tensors on sm_100a, behind tpb200_softmax.
// Replaces cudnn_softmax of p10/src/backend/cuda/ActivationKernels.cu:136-181 (a 4-D padded
// cudnnSoftmaxForward with int dims) with kernels that read the input once from HBM and write the
// output once.  Arithmetic follows the reference's CPU kernels (PointwiseKernels.cpp:519-546):
//   m = max over the dim (the reduction kernels' rule: NaN is never the maximum),
//   e = exp(x - m),  s = sum e,  softmax = e / s,  log_softmax = (x - m) - log s
// with no special cases, so rows holding NaN, +inf or only -inf come out as NaN exactly where the
// reference's chain of float operations produces NaN.  exp is float32 (hardware ex2), the quotient a
// multiplication by the reciprocal of the sum; the sum is kept per thread in float32 over a few
// hundred terms and merged in float64.  Results are held to 1e-5 relative of a float64 evaluation.
//
//   dim is the last, contiguous dim ("rows"):
//     softmax_warp_kernel   one warp per row, the row in registers            (rows of up to 1024)
//     softmax_reg_kernel    one CTA per 16-byte aligned row of 1025 .. 16384 elements, the row in registers
//     softmax_long_kernel   S CTAs per row (a cluster when S > 1): every thread keeps a running
//                           (max, sum) pair over its part, the CTA's pair goes to every CTA of the
//                           row through distributed shared memory, one cluster barrier, and the second
//                           sweep writes the result from the CTA's slice, which stayed in shared memory
//                           (slices of up to 24 K elements; longer ones are read again, from L2 at best)
//   any other dim of a contiguous tensor, viewed as [outer, C, inner]:
//     softmax_col_kernel    a thread per (outer, inner) column, coalesced along inner, two sweeps
#define TPB_FILE_ID 4
#include "common.cuh"
#include "host_util.h"

#include <cooperative_groups.h>

#include <algorithm>

namespace tpb {

namespace cg = cooperative_groups;

// exp on the hot path: ex2.approx of x * log2(e) (two instructions; the library expf and a float
// division per element made the kernels compute-bound: [4096,4096] took 57-61 us with them).  Relative
// error about 2^-22 plus 2^-24 * |x| from the rounded product: below 3e-6 for |x| < 88, inside the 1e-5
// that the results are held to.  exp(-inf) = 0 and exp(NaN) = NaN as with expf.
__device__ __forceinline__ float fast_exp(float x) { return __expf(x); }

// Running (max, sum of exp(x - max)) of a set of values; the empty set is (-inf, 0).
struct MaxSum {
    float m, s;
    __device__ __forceinline__ void init() { m = -INFINITY; s = 0.0f; }
    // four values at once: one rescale of the sum at most
    __device__ __forceinline__ void add4(float a, float b, float c, float d) {
        // the reference's max scan skips NaN (strict compare); fmaxf does the same
        const float cm = fmaxf(fmaxf(a, b), fmaxf(c, d));
        if (cm > m) { s *= fast_exp(m - cm); m = cm; }   // m = -inf, s = 0 at the start: 0 * exp(-inf) = 0
        if (m == -INFINITY) {
            // nothing but -inf (and maybe NaN) so far: -inf adds nothing once the row's maximum is known
            // (exp(-inf - max) = 0); only a NaN must not be lost
            if (a != a || b != b || c != c || d != d) s = NAN;
            return;
        }
        s += (fast_exp(a - m) + fast_exp(b - m)) + (fast_exp(c - m) + fast_exp(d - m));
    }
    // sixteen values at once (the streaming loops of the long rows): one compare against the running
    // maximum and one test for the all -inf start per sixteen elements -- the kernel was bound by
    // instruction issue, not by memory, while it did both per four
    __device__ __forceinline__ void add16(const float4 (&v)[4]) {
        float cm = fmaxf(fmaxf(v[0].x, v[0].y), fmaxf(v[0].z, v[0].w));
#pragma unroll
        for (int u = 1; u < 4; ++u) cm = fmaxf(cm, fmaxf(fmaxf(v[u].x, v[u].y), fmaxf(v[u].z, v[u].w)));
        if (cm > m) { s *= fast_exp(m - cm); m = cm; }
        if (m == -INFINITY) {
            float t = 0.0f;   // -inf and NaN only: the sum is NaN iff one of them is NaN
#pragma unroll
            for (int u = 0; u < 4; ++u) t += (v[u].x + v[u].y) + (v[u].z + v[u].w);
            if (t != t) s = NAN;
            return;
        }
        float t = 0.0f;
#pragma unroll
        for (int u = 0; u < 4; ++u)
            t += (fast_exp(v[u].x - m) + fast_exp(v[u].y - m)) + (fast_exp(v[u].z - m) + fast_exp(v[u].w - m));
        s += t;
    }
    __device__ __forceinline__ void add(float a) {
        if (a > m) { s *= fast_exp(m - a); m = a; }
        if (m == -INFINITY) { if (a != a) s = NAN; return; }
        s += fast_exp(a - m);
    }
};

// Merging the threads' (m, s) pairs: the maximum first (shuffles of one float), then every thread
// brings its sum to that maximum with ONE exp, then the sums are added in float64.  (A tree of pairwise
// merges with an exp at every level put ten dependent float64 exps behind every row.)
//   m = -inf  the thread saw nothing that counts: its s (0, or NaN if it saw a NaN) passes unscaled
//   M = +inf  exp(inf - inf) = NaN, as in the reference's chain
__device__ __forceinline__ float warp_max(float m) {
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) m = fmaxf(m, __shfl_xor_sync(kFull, m, d));
    return m;
}
__device__ __forceinline__ double warp_sum(double s) {
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) s += __shfl_xor_sync(kFull, s, d);
    return s;
}
__device__ __forceinline__ double rescaled(float m, double s, float M) {
    return m == -INFINITY ? s : s * (double)expf(m - M);
}

// ---------------------------------------------------------------- one warp per row ----------
template <bool LOG, int VPL /* float4 per lane */>
__global__ void __launch_bounds__(256)
softmax_warp_kernel(const float* __restrict__ in, float* __restrict__ out, long long rows, long long k1,
                    long long ks0, long long ks1, int len, int vec) {
    const int lane = threadIdx.x & 31;
    const long long r = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (r >= rows) return;
    const long long a = r / k1, b = r - a * k1;
    const float* p = in + a * ks0 + b * ks1;
    float* q = out + r * (long long)len;
    float4 v[VPL];
    MaxSum acc;
    acc.init();
#pragma unroll
    for (int u = 0; u < VPL; ++u) {
        const int e0 = (u * 32 + lane) * 4;
        if (vec && e0 + 3 < len) {
            v[u] = ld_stream4(p + e0);
        } else {
            float t[4];
#pragma unroll
            for (int c = 0; c < 4; ++c) t[c] = e0 + c < len ? ld_stream1(p + e0 + c) : -INFINITY;
            v[u] = make_float4(t[0], t[1], t[2], t[3]);
        }
    }
#pragma unroll
    for (int u = 0; u < VPL; ++u) {
        if ((u * 32 + lane) * 4 < len) acc.add4(v[u].x, v[u].y, v[u].z, v[u].w);   // padding is -inf: exp gives 0
    }
    const float m = warp_max(acc.m);
    const float s = (float)warp_sum(rescaled(acc.m, (double)acc.s, m));
    const float log_s = logf(s), inv_s = 1.0f / s;
#pragma unroll
    for (int u = 0; u < VPL; ++u) {
        const int e0 = (u * 32 + lane) * 4;
        const float o0 = LOG ? (v[u].x - m) - log_s : fast_exp(v[u].x - m) * inv_s;
        const float o1 = LOG ? (v[u].y - m) - log_s : fast_exp(v[u].y - m) * inv_s;
        const float o2 = LOG ? (v[u].z - m) - log_s : fast_exp(v[u].z - m) * inv_s;
        const float o3 = LOG ? (v[u].w - m) - log_s : fast_exp(v[u].w - m) * inv_s;
        if (vec && e0 + 3 < len) {
            *reinterpret_cast<float4*>(TPB_CKN(q + e0, 16)) = make_float4(o0, o1, o2, o3);
        } else {
            if (e0 < len) *TPB_CK(&q[e0]) = o0;
            if (e0 + 1 < len) *TPB_CK(&q[e0 + 1]) = o1;
            if (e0 + 2 < len) *TPB_CK(&q[e0 + 2]) = o2;
            if (e0 + 3 < len) *TPB_CK(&q[e0 + 3]) = o3;
        }
    }
}

// ---------------------------------------------------------------- one CTA per row, row in registers
// Rows of 1025 .. 16384 elements (16-byte aligned, length a multiple of 4): every thread keeps its
// VPT float4 in registers, so the row is read once and the exponentials are computed once.  With
// the whole row at hand the plain chain of the reference is the cheapest form: the maximum (NaN
// skipped, as in the reference's strict compare), e = exp(x - max), the sum, e / sum -- about seven
// instructions per element where the running (max, sum) form with its rescaling and special cases
// needed forty ([4096,4096]: 76 % of the issue slots busy at 27 us).  NaN, +inf and all -inf rows
// come out as NaN through the arithmetic itself: exp(NaN), inf - inf.
template <bool LOG, int VPT>
__global__ void __launch_bounds__(512)
softmax_reg_kernel(const float* __restrict__ in, float* __restrict__ out, long long k1, long long ks0,
                   long long ks1, int len) {
    __shared__ float red_m[16];
    __shared__ float red_s[16];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nthr = blockDim.x, nw = nthr >> 5;
    const long long r = blockIdx.x;
    const long long a = r / k1, b = r - a * k1;
    const float* p = in + a * ks0 + b * ks1;
    float* q = out + r * (long long)len;
    const int nvec = len >> 2;
    float4 v[VPT];
#pragma unroll
    for (int u = 0; u < VPT; ++u) {
        const int i = u * nthr + tid;
        v[u] = i < nvec ? ld_stream4(p + 4 * i) : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
    }
    float m = -INFINITY;
#pragma unroll
    for (int u = 0; u < VPT; ++u) m = fmaxf(m, fmaxf(fmaxf(v[u].x, v[u].y), fmaxf(v[u].z, v[u].w)));
    m = warp_max(m);
    if (lane == 0) red_m[warp] = m;
    __syncthreads();
    m = warp_max(lane < nw ? red_m[lane] : -INFINITY);
    // padding is -inf: exp(-inf - m) = 0 for every m but -inf, and a row of nothing but -inf is NaN anyway
    float s = 0.0f;
#pragma unroll
    for (int u = 0; u < VPT; ++u) {
        const float e0 = fast_exp(v[u].x - m), e1 = fast_exp(v[u].y - m), e2 = fast_exp(v[u].z - m), e3 = fast_exp(v[u].w - m);
        s += (e0 + e1) + (e2 + e3);
        if (!LOG) v[u] = make_float4(e0, e1, e2, e3);
    }
    s = (float)warp_sum((double)s);
    if (lane == 0) red_s[warp] = s;
    __syncthreads();
    s = (float)warp_sum(lane < nw ? (double)red_s[lane] : 0.0);
    const float log_s = logf(s), inv_s = 1.0f / s;
#pragma unroll
    for (int u = 0; u < VPT; ++u) {
        const int i = u * nthr + tid;
        if (i < nvec) {
            float4 o;
            o.x = LOG ? (v[u].x - m) - log_s : v[u].x * inv_s;
            o.y = LOG ? (v[u].y - m) - log_s : v[u].y * inv_s;
            o.z = LOG ? (v[u].z - m) - log_s : v[u].z * inv_s;
            o.w = LOG ? (v[u].w - m) - log_s : v[u].w * inv_s;
            *reinterpret_cast<float4*>(TPB_CKN(q + 4 * i, 16)) = o;
        }
    }
}

// ---------------------------------------------------------------- long rows: S CTAs per row --
// Also serves rows of a few thousand elements with S = 1 (the second sweep then hits L1 / L2).
struct LongShared {
    float wm[32];
    double wsum[32];
    float cm[8];      // (max, sum) of every CTA of the row, written by those CTAs
    double cs[8];
};

// STAGE: the CTA's slice is kept in dynamic shared memory between the two sweeps (the vectorised path
// only, slices of at most 24 K elements), so the input is read from memory exactly once; otherwise the
// second sweep reads it again and relies on L2.
template <bool LOG, bool STAGE>
__global__ void __launch_bounds__(512, 2)
softmax_long_kernel(const float* __restrict__ in, float* __restrict__ out, long long k1, long long ks0,
                    long long ks1, long long len, long long chunk, int S, int vec) {
    extern __shared__ __align__(16) float stage[];
    __shared__ LongShared sh;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nthr = blockDim.x;
    cg::cluster_group cluster = cg::this_cluster();
    const int c = S > 1 ? (int)cluster.block_rank() : 0;
    const long long r = (long long)(blockIdx.x / (unsigned)S);
    const long long a = r / k1, b = r - a * k1;
    const float* row = in + a * ks0 + b * ks1;
    const long long begin = (long long)c * chunk;
    long long n = len - begin;
    if (n > chunk) n = chunk;
    if (n < 0) n = 0;
    const float* p = row + begin;
    float* q = out + r * len + begin;

    // ---- sweep 1: running (max, sum) per thread, four 16-byte loads in flight
    MaxSum acc;
    acc.init();
    const long long nvec = vec ? (n >> 2) : 0;
    {
        long long i = tid;
        for (; i + 3LL * nthr < nvec; i += 4LL * nthr) {
            float4 v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) v[u] = STAGE ? ld_stream4(p + ((i + (long long)u * nthr) << 2)) : ld_keep4(p + ((i + (long long)u * nthr) << 2));
            if (STAGE) {
#pragma unroll
                for (int u = 0; u < 4; ++u) reinterpret_cast<float4*>(stage)[i + (long long)u * nthr] = v[u];
            }
            acc.add16(v);
        }
        for (; i < nvec; i += nthr) {
            const float4 v = STAGE ? ld_stream4(p + (i << 2)) : ld_keep4(p + (i << 2));
            if (STAGE) reinterpret_cast<float4*>(stage)[i] = v;
            acc.add4(v.x, v.y, v.z, v.w);
        }
        for (long long j = (nvec << 2) + tid; j < n; j += nthr) acc.add(*TPB_CK(&p[j]));
    }
    // ---- the CTA's pair (every thread ends up with it), then the row's pair
    const int nw = nthr >> 5;
    const float wmx = warp_max(acc.m);
    if (lane == 0) sh.wm[warp] = wmx;
    __syncthreads();
    float m = warp_max(lane < nw ? sh.wm[lane] : -INFINITY);
    const double wsm = warp_sum(rescaled(acc.m, (double)acc.s, m));
    if (lane == 0) sh.wsum[warp] = wsm;
    __syncthreads();
    double sd = warp_sum(lane < nw ? sh.wsum[lane] : 0.0);
    if (S > 1) {
        if (tid < S) {   // this CTA's pair into every CTA of the row
            *cluster.map_shared_rank(&sh.cm[c], (unsigned)tid) = m;
            *cluster.map_shared_rank(&sh.cs[c], (unsigned)tid) = sd;
        }
        cluster.sync();
        const float cm = lane < S ? sh.cm[lane] : -INFINITY;
        m = warp_max(cm);
        sd = warp_sum(lane < S ? rescaled(cm, sh.cs[lane], m) : 0.0);   // the same order in every CTA
    }
    const float s = (float)sd;
    const float log_s = logf(s), inv_s = 1.0f / s;

    // ---- sweep 2: the slice again (L2), result out
    {
        long long i = tid;
        // four loads in flight per thread here too: the slice comes from L2 at best
        for (; i + 3LL * nthr < nvec; i += 4LL * nthr) {
            float4 v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u)
                v[u] = STAGE ? reinterpret_cast<const float4*>(stage)[i + (long long)u * nthr] : ld_stream4(p + ((i + (long long)u * nthr) << 2));
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                float4 o;
                o.x = LOG ? (v[u].x - m) - log_s : fast_exp(v[u].x - m) * inv_s;
                o.y = LOG ? (v[u].y - m) - log_s : fast_exp(v[u].y - m) * inv_s;
                o.z = LOG ? (v[u].z - m) - log_s : fast_exp(v[u].z - m) * inv_s;
                o.w = LOG ? (v[u].w - m) - log_s : fast_exp(v[u].w - m) * inv_s;
                *reinterpret_cast<float4*>(TPB_CKN(q + ((i + (long long)u * nthr) << 2), 16)) = o;
            }
        }
        for (; i < nvec; i += nthr) {
            const float4 v = STAGE ? reinterpret_cast<const float4*>(stage)[i] : ld_stream4(p + (i << 2));
            float4 o;
            o.x = LOG ? (v.x - m) - log_s : fast_exp(v.x - m) * inv_s;
            o.y = LOG ? (v.y - m) - log_s : fast_exp(v.y - m) * inv_s;
            o.z = LOG ? (v.z - m) - log_s : fast_exp(v.z - m) * inv_s;
            o.w = LOG ? (v.w - m) - log_s : fast_exp(v.w - m) * inv_s;
            *reinterpret_cast<float4*>(TPB_CKN(q + (i << 2), 16)) = o;
        }
        for (long long j = (nvec << 2) + tid; j < n; j += nthr) {
            const float x = *TPB_CK(&p[j]);
            *TPB_CK(&q[j]) = LOG ? (x - m) - log_s : fast_exp(x - m) * inv_s;
        }
    }
    // a CTA must not leave while the others may still write their pair into its shared memory:
    // all remote stores happened before the cluster barrier above, so nothing is needed here
}

// ---------------------------------------------------------------- any other dim --------------
// Contiguous tensor viewed as [outer, C, inner], inner > 1: thread (o, i) walks its column twice.
template <bool LOG>
__global__ void __launch_bounds__(256)
softmax_col_kernel(const float* __restrict__ in, float* __restrict__ out, long long outer, long long C,
                   long long inner) {
    const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= outer * inner) return;
    const long long o = t / inner, i = t - o * inner;
    const float* p = in + o * C * inner + i;
    float* q = out + o * C * inner + i;
    MaxSum acc;
    acc.init();
    long long j = 0;
    for (; j + 3 < C; j += 4) {
        const float x0 = *TPB_CK(&p[j * inner]), x1 = *TPB_CK(&p[(j + 1) * inner]), x2 = *TPB_CK(&p[(j + 2) * inner]), x3 = *TPB_CK(&p[(j + 3) * inner]);
        acc.add4(x0, x1, x2, x3);
    }
    for (; j < C; ++j) acc.add(*TPB_CK(&p[j * inner]));
    const float m = acc.m, log_s = logf(acc.s), inv_s = 1.0f / acc.s;
    for (j = 0; j < C; ++j) {
        const float x = *TPB_CK(&p[j * inner]);
        *TPB_CK(&q[j * inner]) = LOG ? (x - m) - log_s : fast_exp(x - m) * inv_s;
    }
}

}  // namespace tpb

using namespace tpb;

extern "C" int tpb200_softmax(int log, const void* in, int dtype, int ndim, const int64_t* sizes,
                              const int64_t* strides, int dim, void* out, void* stream) {
    if (dtype != TPB200_F32) return fail(TPB200_ERR_UNSUPPORTED, "only float32 input is supported (dtype code %d)", dtype);
    if (ndim < 1 || ndim > TPB200_MAX_DIMS) return fail(TPB200_ERR_UNSUPPORTED, "tensors of rank %d are not supported (1..%d)", ndim, TPB200_MAX_DIMS);
    if (!sizes || !strides) return fail(TPB200_ERR_INVALID, "sizes/strides must not be NULL");
    int d = dim < 0 ? dim + ndim : dim;
    if (d < 0 || d >= ndim) return fail(TPB200_ERR_DIM_RANGE, "Dimension out of range");
    long long numel = 1;
    for (int i = 0; i < ndim; ++i) {
        if (sizes[i] < 0) return fail(TPB200_ERR_INVALID, "negative size in dim %d", i);
        numel *= sizes[i];
    }
    if (numel == 0) return TPB200_OK;
    if (!in || !out) return fail(TPB200_ERR_INVALID, "NULL pointer argument");
    const long long C = sizes[d];
    cudaStream_t st = (cudaStream_t)stream;
    TPB_CHECK_RANGES(st, view_range(in, ndim, sizes, strides, 4), HostRange{out, (size_t)numel * 4});
    const float* x = (const float*)in;
    float* y = (float*)out;

    // is the whole tensor contiguous?
    bool contig = true;
    {
        long long acc = 1;
        for (int i = ndim - 1; i >= 0; --i) {
            if (sizes[i] != 1 && strides[i] != acc) contig = false;
            acc *= sizes[i];
        }
    }
    long long inner = 1;
    for (int i = d + 1; i < ndim; ++i) inner *= sizes[i];

    if (inner == 1 && (C == 1 || strides[d] == 1)) {
        // rows: the other dims merged where the strides allow; at most two may survive
        struct KD { long long size, stride; };
        KD kept[TPB200_MAX_DIMS];
        int nk = 0;
        long long rows = 1;
        for (int i = 0; i < ndim; ++i) {
            if (i == d) continue;
            rows *= sizes[i];
            if (sizes[i] == 1) continue;
            if (nk > 0 && kept[nk - 1].stride == strides[i] * sizes[i]) { kept[nk - 1].size *= sizes[i]; kept[nk - 1].stride = strides[i]; }
            else { kept[nk].size = sizes[i]; kept[nk].stride = strides[i]; ++nk; }
        }
        if (nk > 2) return fail(TPB200_ERR_UNSUPPORTED, "softmax needs the other dims to collapse to at most two strided dims");
        long long k1 = 1, ks0 = 0, ks1 = 0;
        if (nk == 2) { k1 = kept[1].size; ks0 = kept[0].stride; ks1 = kept[1].stride; }
        else if (nk == 1) { ks0 = kept[0].stride; }
        // 16-byte loads and stores need aligned rows on both sides
        const int vec = (((uintptr_t)in) & 15) == 0 && (((uintptr_t)out) & 15) == 0 && ks0 % 4 == 0 && ks1 % 4 == 0 && C % 4 == 0;
        if (C <= 1024) {
            const int wpc = 8;
            if (ceil_div(rows, wpc) > 0x7fffffffLL) return fail(TPB200_ERR_UNSUPPORTED, "too many rows for one launch");
            const dim3 grid((unsigned)ceil_div(rows, wpc));
#define TPB_SM_WARP(V)                                                                                       \
    do {                                                                                                     \
        if (log) TPB_LAUNCH("softmax_warp_kernel", (softmax_warp_kernel<true, V>), grid, wpc * 32, 0, st, x, y, rows, k1, ks0, ks1, (int)C, vec); \
        else     TPB_LAUNCH("softmax_warp_kernel", (softmax_warp_kernel<false, V>), grid, wpc * 32, 0, st, x, y, rows, k1, ks0, ks1, (int)C, vec); \
    } while (0)
            if (C <= 128) TPB_SM_WARP(1); else if (C <= 256) TPB_SM_WARP(2); else if (C <= 512) TPB_SM_WARP(4); else TPB_SM_WARP(8);
#undef TPB_SM_WARP
            return TPB200_OK;
        }
        if (vec && C <= 16384) {
            // threads so that a thread holds at most four float4 (eight above 8192 elements)
            int threads = 128;
            while (threads < 512 && (long long)threads * 16 < C) threads *= 2;
            if (rows > 0x7fffffffLL) return fail(TPB200_ERR_UNSUPPORTED, "too many rows for one launch");
            const dim3 grid((unsigned)rows);
            const bool v8 = (long long)threads * 16 < C;
#define TPB_SM_REG(LOGV, V) TPB_LAUNCH("softmax_reg_kernel", (softmax_reg_kernel<LOGV, V>), grid, threads, 0, st, x, y, k1, ks0, ks1, (int)C)
            if (log) { if (v8) TPB_SM_REG(true, 8); else TPB_SM_REG(true, 4); }
            else     { if (v8) TPB_SM_REG(false, 8); else TPB_SM_REG(false, 4); }
#undef TPB_SM_REG
            return TPB200_OK;
        }
        // Rows of up to 48 K elements: one or two CTAs per row, each keeping its slice (at most 24 K
        // elements, 96 KB: two CTAs per SM) in shared memory between the sweeps, so the input is read
        // once.  Longer rows: the second sweep reads the slice again, and S only has to give the GPU
        // enough CTAs (two per SM).  Measured on [256,151936] (algorithmic 311 MB, four inputs in
        // rotation): S = 8 with staged slices 84 us -- seven waves of CTAs that each load, wait for
        // their cluster and only then store; S = 1 / 2 / 4 without staging 79 / 72 / 76 us.  72 us is
        // what two reads and one write of the tensor (467 MB) take at the copy bandwidth: with 512 CTAs
        // sweeping 304 KB each the second sweep finds little of its slice left in L2.
        constexpr long long kStageMax = 24 * 1024;
        int S = 1;
        if (C > kStageMax && C <= 2 * kStageMax) S = 2;
        else if (C > 2 * kStageMax)
            while (S < 8 && rows * S < 2LL * sm_count() && ceil_div(C, 2 * S) >= 16384) S *= 2;
        int fs = 0;
        if (env_int("TPB200_SOFTMAX_SLICES", &fs) && (fs == 1 || fs == 2 || fs == 4 || fs == 8)) S = fs;
        const long long chunk = round_up(ceil_div(C, S), 4);
        if (rows * S > 0x7fffffffLL) return fail(TPB200_ERR_UNSUPPORTED, "too many rows for one launch");
        const int threads = C / S >= 8192 ? 512 : (C / S >= 2048 ? 256 : 128);
        const dim3 grid((unsigned)(rows * S));
        int stage_on = 1;
        // experiment switch: 0 never keeps the slice in shared memory ([256,151936] with eight CTAs per row:
        // 84 us staged, 91 us not -- the clusters of eight cost more than the second read saves either way)
        env_int("TPB200_SOFTMAX_STAGE", &stage_on);
        const bool stage = vec && chunk <= kStageMax && stage_on != 0;
        const size_t smem = stage ? (size_t)chunk * sizeof(float) : 0;
        cudaError_t e = cudaSuccess;
#define TPB_SM_LONG(LOGV, STAGEV)                                                                                  \
    do {                                                                                                           \
        if (smem + 8192 > 48 * 1024)                                                                               \
            TPB_CUDA_OK(cudaFuncSetAttribute(softmax_long_kernel<LOGV, STAGEV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
        e = launch_ex(softmax_long_kernel<LOGV, STAGEV>, grid, threads, smem, st, S, false, x, y, k1, ks0, ks1, C, chunk, S, vec);        \
    } while (0)
        if (log) { if (stage) TPB_SM_LONG(true, true); else TPB_SM_LONG(true, false); }
        else     { if (stage) TPB_SM_LONG(false, true); else TPB_SM_LONG(false, false); }
#undef TPB_SM_LONG
        if (e != cudaSuccess) return cuda_fail(e, "softmax_long_kernel");
        return TPB200_OK;
    }
    if (!contig) return fail(TPB200_ERR_UNSUPPORTED, "softmax over a dim other than the last needs a contiguous tensor");
    long long outer = 1;
    for (int i = 0; i < d; ++i) outer *= sizes[i];
    const long long cols = outer * inner;
    if (ceil_div(cols, 256) > 0x7fffffffLL) return fail(TPB200_ERR_UNSUPPORTED, "too many columns for one launch");
    const dim3 grid((unsigned)ceil_div(cols, 256));
    if (log) TPB_LAUNCH("softmax_col_kernel", softmax_col_kernel<true>, grid, 256, 0, st, x, y, outer, C, inner);
    else     TPB_LAUNCH("softmax_col_kernel", softmax_col_kernel<false>, grid, 256, 0, st, x, y, outer, C, inner);
    return TPB200_OK;
}
