// Strided copy of 4-byte elements on sm_100a, behind tpb200_strided_copy: dst[i...] = src[i...] for
// two views of the same shape with arbitrary strides.  Replaces copy_cast_kernel_impl of
// p10/src/backend/cuda/CopyKernels.cu:42-53, 105-156 for the case callers hit around reductions
// (permute().contiguous(), slices, transposes of float32 tensors: ReductionKernels.cu:67-75, 143):
// that kernel moves one element per thread and pays a div/mod chain over all dims per element on
// both sides, and whichever side is not walked along its unit stride is accessed uncoalesced.
//
// The host merges dims that are contiguous in BOTH views and picks one of three kernels:
//   rows     both views have unit stride along the innermost dim: 16-byte loads and stores along it
//            where both sides are aligned, the outer index decoded once per row chunk
//   tiles    the unit strides lie along DIFFERENT dims (a transpose): 64 x 64 tiles through shared
//            memory, read along the source's unit-stride dim, written along the destination's, both
//            coalesced; the other dims are decoded once per tile
//   generic  one element per thread with the div/mod walk, for whatever is left (no unit stride)
#define TPB_FILE_ID 6
#include "common.cuh"
#include "host_util.h"

#include <algorithm>

namespace tpb {

struct CopyGeom {
    int nd;                                   // merged dims, outermost first
    long long size[TPB200_MAX_DIMS], ds[TPB200_MAX_DIMS], ss[TPB200_MAX_DIMS];
};

// ---- rows: innermost dim contiguous on both sides
template <int VEC>
__global__ void __launch_bounds__(256)
copy_rows_kernel(unsigned* __restrict__ dst, const unsigned* __restrict__ src, CopyGeom g, long long chunks_per_row,
                 long long total_chunks) {
    const int nd = g.nd;
    const long long len = g.size[nd - 1];
    for (long long c = blockIdx.x; c < total_chunks; c += gridDim.x) {
        long long row = c / chunks_per_row;
        const long long ch = c - row * chunks_per_row;
        long long doff = 0, soff = 0;
        for (int d = nd - 2; d >= 0; --d) {
            const long long i = row % g.size[d];
            row /= g.size[d];
            doff += i * g.ds[d];
            soff += i * g.ss[d];
        }
        const long long e0 = ch * (256LL * 4 * VEC);      // 256 threads x 4 vectors per chunk
        const unsigned* s = src + soff;
        unsigned* t = dst + doff;
        if (VEC == 4) {
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const long long e = e0 + ((long long)u * 256 + threadIdx.x) * 4;
                if (e + 3 < len) {
                    const uint4 v = *reinterpret_cast<const uint4*>(TPB_CKN(s + e, 16));
                    *reinterpret_cast<uint4*>(TPB_CKN(t + e, 16)) = v;
                } else {
                    for (long long q = e; q < len && q < e + 4; ++q) *TPB_CK(&t[q]) = *TPB_CK(&s[q]);
                }
            }
        } else {
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const long long e = e0 + (long long)u * 256 + threadIdx.x;
                if (e < len) *TPB_CK(&t[e]) = *TPB_CK(&s[e]);
            }
        }
    }
}

// ---- tiles: dim A has unit stride in src, dim B has unit stride in dst.  64 x 64 tiles: a thread has
// sixteen 4-byte loads in flight (a 32 x 32 tile with four per thread moved 2.75 TB/s on
// [64,4096,512] -> [64,512,4096]: too few bytes in flight per SM).
constexpr int kTile = 64;
__global__ void __launch_bounds__(256)
copy_tiles_kernel(unsigned* __restrict__ dst, const unsigned* __restrict__ src, CopyGeom g, int A, int B,
                  long long tiles_a, long long tiles_b, long long total_tiles) {
    __shared__ unsigned tile[kTile][kTile + 1];
    const int tx = threadIdx.x & 63, ty = threadIdx.x >> 6;    // 64 x 4
    for (long long t = blockIdx.x; t < total_tiles; t += gridDim.x) {
        long long rest = t / (tiles_a * tiles_b);
        const long long tt = t - rest * (tiles_a * tiles_b);
        const long long tb = tt / tiles_a, ta = tt - tb * tiles_a;
        long long doff = 0, soff = 0;
        for (int d = g.nd - 1; d >= 0; --d) {
            if (d == A || d == B) continue;
            const long long i = rest % g.size[d];
            rest /= g.size[d];
            doff += i * g.ds[d];
            soff += i * g.ss[d];
        }
        const long long a0 = ta * kTile, b0 = tb * kTile;
        // Addresses by pointer increments and no bounds tests on full tiles: with a 64-bit multiply and
        // two 64-bit compares per element the kernel was bound by instruction issue (82 % of the issue
        // slots busy at 74 % of the copy bandwidth).
        const bool full = a0 + kTile <= g.size[A] && b0 + kTile <= g.size[B];
        unsigned v[16];
        {
            const long long a = a0 + tx;
            const long long step = 4 * g.ss[B];
            const unsigned* p = src + soff + a * g.ss[A] + (b0 + ty) * g.ss[B];
            if (full) {
#pragma unroll
                for (int j = 0; j < 16; ++j) v[j] = *TPB_CK(p + j * step);
            } else {
#pragma unroll
                for (int j = 0; j < 16; ++j) v[j] = (a < g.size[A] && b0 + ty + 4 * j < g.size[B]) ? *TPB_CK(p + j * step) : 0u;
            }
#pragma unroll
            for (int j = 0; j < 16; ++j) tile[ty + 4 * j][tx] = v[j];
        }
        __syncthreads();
        {
            const long long b = b0 + tx;
            const long long step = 4 * g.ds[A];
            unsigned* q = dst + doff + b * g.ds[B] + (a0 + ty) * g.ds[A];
            if (full) {
#pragma unroll
                for (int j = 0; j < 16; ++j) *TPB_CK(q + j * step) = tile[tx][ty + 4 * j];
            } else {
#pragma unroll
                for (int j = 0; j < 16; ++j)
                    if (a0 + ty + 4 * j < g.size[A] && b < g.size[B]) *TPB_CK(q + j * step) = tile[tx][ty + 4 * j];
            }
        }
        __syncthreads();
    }
}

// ---- generic
__global__ void __launch_bounds__(256)
copy_generic_kernel(unsigned* __restrict__ dst, const unsigned* __restrict__ src, CopyGeom g, long long numel) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < numel; i += (long long)gridDim.x * blockDim.x) {
        long long q = i, doff = 0, soff = 0;
        for (int d = g.nd - 1; d >= 0; --d) {
            const long long c = q % g.size[d];
            q /= g.size[d];
            doff += c * g.ds[d];
            soff += c * g.ss[d];
        }
        *TPB_CK(&dst[doff]) = *TPB_CK(&src[soff]);
    }
}

}  // namespace tpb

using namespace tpb;

extern "C" int tpb200_strided_copy(void* dst, const int64_t* dst_strides, const void* src, const int64_t* src_strides,
                                   int dtype, int ndim, const int64_t* sizes, void* stream) {
    if (dtype != TPB200_F32) return fail(TPB200_ERR_UNSUPPORTED, "only 4-byte elements (dtype code %d) are copied", TPB200_F32);
    if (ndim < 0 || ndim > TPB200_MAX_DIMS) return fail(TPB200_ERR_UNSUPPORTED, "tensors of rank %d are not supported (max %d)", ndim, TPB200_MAX_DIMS);
    if (ndim > 0 && (!sizes || !dst_strides || !src_strides)) return fail(TPB200_ERR_INVALID, "sizes/strides must not be NULL");
    long long numel = 1;
    CopyGeom g{};
    for (int i = 0; i < ndim; ++i) {
        if (sizes[i] < 0) return fail(TPB200_ERR_INVALID, "negative size in dim %d", i);
        numel *= sizes[i];
        if (sizes[i] == 1) continue;
        // merge with the previous dim where both views run on without a gap
        if (g.nd > 0 && g.ds[g.nd - 1] == dst_strides[i] * sizes[i] && g.ss[g.nd - 1] == src_strides[i] * sizes[i]) {
            g.size[g.nd - 1] *= sizes[i];
            g.ds[g.nd - 1] = dst_strides[i];
            g.ss[g.nd - 1] = src_strides[i];
        } else {
            g.size[g.nd] = sizes[i];
            g.ds[g.nd] = dst_strides[i];
            g.ss[g.nd] = src_strides[i];
            ++g.nd;
        }
    }
    if (numel == 0) return TPB200_OK;
    if (!dst || !src) return fail(TPB200_ERR_INVALID, "NULL pointer argument");
    if (g.nd == 0) { g.nd = 1; g.size[0] = 1; g.ds[0] = 1; g.ss[0] = 1; }
    cudaStream_t st = (cudaStream_t)stream;
    TPB_CHECK_RANGES(st, view_range(src, ndim, sizes, src_strides, 4), view_range(dst, ndim, sizes, dst_strides, 4));
    unsigned* d = (unsigned*)dst;
    const unsigned* s = (const unsigned*)src;
    const int sms = sm_count();
    const int last = g.nd - 1;
    if (g.ds[last] == 1 && g.ss[last] == 1) {
        const long long len = g.size[last];
        bool vec = ((((uintptr_t)dst) | ((uintptr_t)src)) & 15) == 0;
        for (int i = 0; i < last; ++i) vec = vec && g.ds[i] % 4 == 0 && g.ss[i] % 4 == 0;
        const long long per_chunk = vec ? 256LL * 16 : 256LL * 4;
        const long long chunks_per_row = ceil_div(len, per_chunk);
        const long long total = (numel / len) * chunks_per_row;
        const dim3 grid((unsigned)std::min<long long>(total, (long long)sms * 32));
        if (vec) TPB_LAUNCH("copy_rows_kernel", copy_rows_kernel<4>, grid, 256, 0, st, d, s, g, chunks_per_row, total);
        else     TPB_LAUNCH("copy_rows_kernel", copy_rows_kernel<1>, grid, 256, 0, st, d, s, g, chunks_per_row, total);
        return TPB200_OK;
    }
    int A = -1, B = -1;
    for (int i = 0; i < g.nd; ++i) {
        if (g.ss[i] == 1 && A < 0) A = i;
        if (g.ds[i] == 1 && B < 0) B = i;
    }
    if (A >= 0 && B >= 0 && A != B) {
        const long long ta = ceil_div(g.size[A], kTile), tb = ceil_div(g.size[B], kTile);
        const long long total = (numel / (g.size[A] * g.size[B])) * ta * tb;
        const dim3 grid((unsigned)std::min<long long>(total, (long long)sms * 64));
        TPB_LAUNCH("copy_tiles_kernel", copy_tiles_kernel, grid, 256, 0, st, d, s, g, A, B, ta, tb, total);
        return TPB200_OK;
    }
    const dim3 grid((unsigned)std::min<long long>(ceil_div(numel, 256), (long long)sms * 64));
    TPB_LAUNCH("copy_generic_kernel", copy_generic_kernel, grid, 256, 0, st, d, s, g, numel);
    return TPB200_OK;
}
