// softmax / log_softmax along one dim for float32 tensors on sm_100a, behind tpb200_softmax.
// Replaces cudnn_softmax of p10/src/backend/cuda/ActivationKernels.cu:136-181 (a 4-D padded
// cudnnSoftmaxForward with int dims) with kernels that read the input once from HBM and write the
// output once.  Arithmetic follows the reference's CPU kernels (PointwiseKernels.cpp:519-546):
//   m = max over the dim (the reduction kernels' rule: NaN is never the maximum),
//   e = exp(x - m),  s = sum e,  softmax = e / s,  log_softmax = (x - m) - log s
// with no special cases, so rows holding NaN, +inf or only -inf come out as NaN exactly where the
// reference's chain of float operations produces NaN.  exp and the quotient are float32; the sum is
// kept per thread in float32 over a few hundred terms and merged in float64.
//
//   dim is the last, contiguous dim ("rows"):
//     softmax_warp_kernel   one warp per row, the row in registers            (rows of up to 1024)
//     softmax_long_kernel   S CTAs per row (a cluster when S > 1): every thread keeps a running
//                           (max, sum) pair over its part, the CTA's pair goes to every CTA of the
//                           row through distributed shared memory, one cluster barrier, and the second
//                           sweep over the CTA's slice -- still in L2 -- writes the result
//   any other dim of a contiguous tensor, viewed as [outer, C, inner]:
//     softmax_col_kernel    a thread per (outer, inner) column, coalesced along inner, two sweeps
#include "common.cuh"
#include "host_util.h"

#include <cooperative_groups.h>

#include <algorithm>

namespace tpb {

namespace cg = cooperative_groups;

// Running (max, sum of exp(x - max)) of a set of values; the empty set is (-inf, 0).
struct MaxSum {
    float m, s;
    __device__ __forceinline__ void init() { m = -INFINITY; s = 0.0f; }
    // four values at once: one rescale of the sum at most
    __device__ __forceinline__ void add4(float a, float b, float c, float d) {
        // the reference's max scan skips NaN (strict compare); fmaxf does the same
        const float cm = fmaxf(fmaxf(a, b), fmaxf(c, d));
        if (cm > m) { s *= expf(m - cm); m = cm; }   // m = -inf, s = 0 at the start: 0 * exp(-inf) = 0
        if (m == -INFINITY) {
            // nothing but -inf (and maybe NaN) so far: -inf adds nothing once the row's maximum is known
            // (exp(-inf - max) = 0); only a NaN must not be lost
            if (a != a || b != b || c != c || d != d) s = NAN;
            return;
        }
        s += (expf(a - m) + expf(b - m)) + (expf(c - m) + expf(d - m));
    }
    __device__ __forceinline__ void add(float a) {
        if (a > m) { s *= expf(m - a); m = a; }
        if (m == -INFINITY) { if (a != a) s = NAN; return; }
        s += expf(a - m);
    }
};

// Merge in float64: (m, s) pairs of lanes, warps, CTAs.  NaN sums propagate; a part that saw
// nothing (m = -inf, s = 0) leaves the other unchanged.
struct MaxSum64 {
    float m;
    double s;
    __device__ __forceinline__ void merge(float om, double os) {
        if (om > m) { s = s * exp((double)m - (double)om) + os; m = om; }
        else if (om == m) { s += os; }
        else { s += os * exp((double)om - (double)m); }
    }
};

__device__ __forceinline__ MaxSum64 warp_merge(float m, double s) {
    MaxSum64 r{m, s};
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
        const float om = __shfl_xor_sync(kFull, r.m, d);
        const double os = __shfl_xor_sync(kFull, r.s, d);
        // both partners must end up with the same pair: merge symmetrically
        MaxSum64 t = r;
        t.merge(om, os);
        r = t;
    }
    return r;
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
    const MaxSum64 t = warp_merge(acc.m, (double)acc.s);
    const float m = t.m, s = (float)t.s;
    const float log_s = logf(s);
#pragma unroll
    for (int u = 0; u < VPL; ++u) {
        const int e0 = (u * 32 + lane) * 4;
        const float o0 = LOG ? (v[u].x - m) - log_s : expf(v[u].x - m) / s;
        const float o1 = LOG ? (v[u].y - m) - log_s : expf(v[u].y - m) / s;
        const float o2 = LOG ? (v[u].z - m) - log_s : expf(v[u].z - m) / s;
        const float o3 = LOG ? (v[u].w - m) - log_s : expf(v[u].w - m) / s;
        if (vec && e0 + 3 < len) {
            *reinterpret_cast<float4*>(q + e0) = make_float4(o0, o1, o2, o3);
        } else {
            if (e0 < len) q[e0] = o0;
            if (e0 + 1 < len) q[e0 + 1] = o1;
            if (e0 + 2 < len) q[e0 + 2] = o2;
            if (e0 + 3 < len) q[e0 + 3] = o3;
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
    float m;
    float s;
};

template <bool LOG>
__global__ void __launch_bounds__(512, 2)
softmax_long_kernel(const float* __restrict__ in, float* __restrict__ out, long long k1, long long ks0,
                    long long ks1, long long len, long long chunk, int S, int vec) {
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
            for (int u = 0; u < 4; ++u) v[u] = ld_keep4(p + ((i + (long long)u * nthr) << 2));
#pragma unroll
            for (int u = 0; u < 4; ++u) acc.add4(v[u].x, v[u].y, v[u].z, v[u].w);
        }
        for (; i < nvec; i += nthr) {
            const float4 v = ld_keep4(p + (i << 2));
            acc.add4(v.x, v.y, v.z, v.w);
        }
        for (long long j = (nvec << 2) + tid; j < n; j += nthr) acc.add(p[j]);
    }
    // ---- CTA pair, then the row's pair
    MaxSum64 t = warp_merge(acc.m, (double)acc.s);
    if (lane == 0) { sh.wm[warp] = t.m; sh.wsum[warp] = t.s; }
    __syncthreads();
    if (warp == 0) {
        const int nw = nthr >> 5;
        MaxSum64 u = warp_merge(lane < nw ? sh.wm[lane] : -INFINITY, lane < nw ? sh.wsum[lane] : 0.0);
        if (lane == 0) {
            if (S > 1) {
                for (int j = 0; j < S; ++j) {   // this CTA's pair into every CTA of the row
                    *cluster.map_shared_rank(&sh.cm[c], (unsigned)j) = u.m;
                    *cluster.map_shared_rank(&sh.cs[c], (unsigned)j) = u.s;
                }
            } else {
                sh.m = u.m;
                sh.s = (float)u.s;
            }
        }
    }
    if (S > 1) {
        cluster.sync();
        if (tid == 0) {
            MaxSum64 u{sh.cm[0], sh.cs[0]};
            for (int j = 1; j < S; ++j) u.merge(sh.cm[j], sh.cs[j]);   // the same order in every CTA
            sh.m = u.m;
            sh.s = (float)u.s;
        }
    }
    __syncthreads();
    const float m = sh.m, s = sh.s;
    const float log_s = logf(s);

    // ---- sweep 2: the slice again (L2), result out
    {
        long long i = tid;
        for (; i < nvec; i += nthr) {
            const float4 v = ld_stream4(p + (i << 2));
            float4 o;
            o.x = LOG ? (v.x - m) - log_s : expf(v.x - m) / s;
            o.y = LOG ? (v.y - m) - log_s : expf(v.y - m) / s;
            o.z = LOG ? (v.z - m) - log_s : expf(v.z - m) / s;
            o.w = LOG ? (v.w - m) - log_s : expf(v.w - m) / s;
            *reinterpret_cast<float4*>(q + (i << 2)) = o;
        }
        for (long long j = (nvec << 2) + tid; j < n; j += nthr) {
            const float x = p[j];
            q[j] = LOG ? (x - m) - log_s : expf(x - m) / s;
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
        const float x0 = p[j * inner], x1 = p[(j + 1) * inner], x2 = p[(j + 2) * inner], x3 = p[(j + 3) * inner];
        acc.add4(x0, x1, x2, x3);
    }
    for (; j < C; ++j) acc.add(p[j * inner]);
    const float m = acc.m, s = acc.s, log_s = logf(acc.s);
    for (j = 0; j < C; ++j) {
        const float x = p[j * inner];
        q[j * inner] = LOG ? (x - m) - log_s : expf(x - m) / s;
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
        // S CTAs per row: a cluster of 2, 4 or 8 where the rows alone leave the GPU partly empty and a
        // slice still holds 32 K elements
        const int sms = sm_count();
        int S = 1;
        while (S < 8 && rows * (2LL * S) <= 2LL * sms && C / (2LL * S) >= 32 * 1024) S *= 2;
        int fs = 0;
        if (env_int("TPB200_SOFTMAX_SLICES", &fs) && (fs == 1 || fs == 2 || fs == 4 || fs == 8)) S = fs;
        const long long chunk = round_up(ceil_div(C, S), 4);
        if (rows * S > 0x7fffffffLL) return fail(TPB200_ERR_UNSUPPORTED, "too many rows for one launch");
        const int threads = C / S >= 8192 ? 512 : (C / S >= 2048 ? 256 : 128);
        const dim3 grid((unsigned)(rows * S));
        cudaError_t e;
        if (log) e = launch_ex(softmax_long_kernel<true>, grid, threads, 0, st, S, false, x, y, k1, ks0, ks1, C, chunk, S, vec);
        else     e = launch_ex(softmax_long_kernel<false>, grid, threads, 0, st, S, false, x, y, k1, ks0, ks1, C, chunk, S, vec);
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
