// Shared device-side building blocks of the sm_100a reduction and top-k kernels:
// streaming 128-bit loads, the three accumulator families (fp64 sum, Welford/Chan moments,
// first-occurrence extremum) with their warp- and block-level combines, and the packed
// partial record exchanged between kernel passes and between GPUs.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <math.h>

#include "../../include/tpb200.h"

namespace tpb {

constexpr int kWarp = 32;
constexpr unsigned kFull = 0xffffffffu;
// "no element selected yet" index: larger than any real position, so a real tie always wins.
constexpr long long kNoIndex = 0x7fffffffffffffffLL;

// ------------------------------------------------------------------ checked build ----------
// With -DTPB200_CHECKED (the library libtpb200_checked.so) every access to global memory goes through
// TPB_CK / TPB_CKN: the address range is compared with the ranges that the host entry point registered
// for its call (input view, outputs, workspace, exchange buffers).  An access outside them is NOT
// made: it is turned to a small sink buffer, the first one is recorded (file id, line, address, size)
// and counted, and the per-device status word becomes kErrChecked.  Nothing traps.  This is the
// stand-in for a memory checker on machines where none can be run; the ordinary build compiles the
// macros to the bare pointer.
constexpr int kErrChecked = 0x40000000;   // above every wait code, so atomicMax keeps it
#ifdef TPB200_CHECKED
constexpr int kCheckRanges = 24;
struct CheckRange { unsigned long long lo, hi; };   // [lo, hi), bytes
struct CheckTable { CheckRange r[kCheckRanges]; int n; int pad; };
struct CheckRecord { int hit, file, line; unsigned bytes; unsigned long long addr, count; };
extern __device__ CheckTable g_check_table;
extern __device__ CheckRecord g_check_record;
extern __device__ __align__(16) unsigned char g_check_sink[256];
__device__ const void* check_access(const void* p, unsigned bytes, int file, int line);
template <class T>
__device__ __forceinline__ T* checked(T* p, unsigned bytes, int file, int line) {
    return (T*)check_access((const void*)p, bytes, file, line);
}
#ifndef TPB_FILE_ID
#define TPB_FILE_ID 0
#endif
#define TPB_CK(p) ::tpb::checked((p), (unsigned)sizeof(*(p)), TPB_FILE_ID, __LINE__)
#define TPB_CKN(p, bytes) ::tpb::checked((p), (unsigned)(bytes), TPB_FILE_ID, __LINE__)
#else
#define TPB_CK(p) (p)
#define TPB_CKN(p, bytes) (p)
#endif

// ------------------------------------------------------------------ loads ------------------
// Input is read exactly once: bypass L1 allocation so the 16-byte sectors stream from L2/HBM.
__device__ __forceinline__ float4 ld_stream4_raw(const float* p) {
    float4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                 : "l"(p));
    return v;
}
// The same 128-bit read-only load WITH allocation in L1: for data that the same SM reads again within
// microseconds (the top-k kernels re-read the few elements that pass their threshold test).
__device__ __forceinline__ float4 ld_keep4_raw(const float* p) {
    float4 v;
    asm volatile("ld.global.nc.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                 : "l"(p));
    return v;
}
__device__ __forceinline__ float ld_stream1_raw(const float* p) {
    float v;
    asm volatile("ld.global.nc.L1::no_allocate.f32 %0, [%1];" : "=f"(v) : "l"(p));
    return v;
}
// the loads as the kernels spell them (macros, so that a checked build records the caller's line)
#define ld_stream4(p) ::tpb::ld_stream4_raw(TPB_CKN((p), 16))
#define ld_keep4(p) ::tpb::ld_keep4_raw(TPB_CKN((p), 16))
#define ld_stream1(p) ::tpb::ld_stream1_raw(TPB_CKN((p), 4))

// ------------------------------------------------------------------ packed partial ---------
// One record per (row, slice) between the two passes of a split reduction, and per GPU in the
// sharded whole-tensor path (it is the all-gather payload).  Field use by family:
//   sum/mean : d0 = sum
//   var/std  : d0 = count, d1 = mean, d2 = M2 (sum of squared deviations from the mean)
//   extremum : f0 = value, i0 = position (kNoIndex when nothing compared better)
struct __align__(8) Packed {
    double d0, d1, d2;
    long long i0;
    float f0;
    unsigned int pad;
};
static_assert(sizeof(Packed) == TPB200_PARTIAL_BYTES, "Packed layout is part of the C ABI");

// ------------------------------------------------------------------ accumulators -----------
// fp64 running sum: every float is widened before the add, so the result is the correctly
// rounded sum up to ~1e-16 relative to sum|x| -- that is what keeps near-zero row sums within
// 1e-5 relative of a float64 evaluation.
struct SumAcc {
    double s;
    __device__ __forceinline__ void init() { s = 0.0; }
    __device__ __forceinline__ void add(float x, long long) { s += (double)x; }
    // four elements at positions pos, pos + step, ...
    __device__ __forceinline__ void add4(float x0, float x1, float x2, float x3, long long pos, long long step) {
        add(x0, pos); add(x1, pos + step); add(x2, pos + 2 * step); add(x3, pos + 3 * step);
    }
    __device__ __forceinline__ void finish_thread() {}
    __device__ __forceinline__ void merge(const SumAcc& o) { s += o.s; }
    __device__ __forceinline__ SumAcc shfl_down(int d) const {
        SumAcc r; r.s = __shfl_down_sync(kFull, s, d); return r;
    }
    __device__ __forceinline__ void store(Packed* p) const { p->d0 = s; p->d1 = 0; p->d2 = 0; p->i0 = 0; p->f0 = 0; p->pad = 0; }
    __device__ __forceinline__ void load(const Packed* p) { s = p->d0; }
};

// Variance.  Inside one thread: moments of d = x - K, K = the thread's first element (shifted-data
// form: no per-element division, and an offset common to the data is gone before anything is
// squared; d is exact in fp32 whenever x and K are within a factor of two of each other).  The
// streaming loops hand over four elements at a time: their d and d*d are summed in fp32 and then
// added to fp64 totals, so the fp64 pipe -- which bounded this kernel when every element went
// through it -- sees a quarter of the work; a sum of four fp32 terms carries a relative error of
// about 1e-7, inside the 1e-5 that the result is held to.  finish_thread() turns the totals into a
// Welford triple (count, mean, M2); everything above a thread -- lanes, warps, CTAs, slices, GPUs
// -- is combined with Chan's pairwise update in fp64, always in a fixed order.
struct MomAcc {
    double n, mean, m2;   // after finish_thread(): count, mean, M2;  before: mean = sum d, m2 = sum d*d
    float kf;             // shift
    unsigned int c;       // elements seen by this thread
    __device__ __forceinline__ void init() { n = 0.0; mean = 0.0; m2 = 0.0; kf = 0.0f; c = 0u; }
    __device__ __forceinline__ void add(float x, long long) {
        if (c == 0u) kf = x;
        const double d = (double)(x - kf);
        ++c;
        mean += d;
        m2 = fma(d, d, m2);
    }
    __device__ __forceinline__ void add4(float x0, float x1, float x2, float x3, long long, long long) {
        if (c == 0u) kf = x0;
        c += 4u;
        const float d0 = x0 - kf, d1 = x1 - kf, d2 = x2 - kf, d3 = x3 - kf;
        mean += (double)((d0 + d1) + (d2 + d3));
        m2 += (double)fmaf(d3, d3, fmaf(d2, d2, fmaf(d1, d1, d0 * d0)));
    }
    __device__ __forceinline__ void finish_thread() {
        n = (double)c;
        if (c > 0u) {
            const double s1 = mean;
            const double inv = 1.0 / n;
            mean = fma(s1, inv, (double)kf);
            m2 = m2 - s1 * s1 * inv;
            if (m2 < 0.0) m2 = 0.0;
        }
    }
    // Chan's pairwise update.  Equal counts -- every level of a tree over threads that saw the same
    // number of elements -- need no division at all.
    __device__ __forceinline__ void merge(const MomAcc& o) {
        if (o.n == 0.0) return;
        if (n == 0.0) { n = o.n; mean = o.mean; m2 = o.m2; return; }
        const double delta = o.mean - mean;
        if (n == o.n) {
            mean = fma(delta, 0.5, mean);
            m2 = m2 + o.m2 + delta * delta * (n * 0.5);
            n = n + n;
            return;
        }
        const double nt = n + o.n;
        const double w = o.n / nt;
        mean = fma(delta, w, mean);
        m2 = m2 + o.m2 + delta * delta * n * w;
        n = nt;
    }
    __device__ __forceinline__ MomAcc shfl_down(int d) const {
        MomAcc r;
        r.n = __shfl_down_sync(kFull, n, d);
        r.mean = __shfl_down_sync(kFull, mean, d);
        r.m2 = __shfl_down_sync(kFull, m2, d);
        r.kf = 0.0f;
        r.c = 0u;
        return r;
    }
    __device__ __forceinline__ void store(Packed* p) const { p->d0 = n; p->d1 = mean; p->d2 = m2; p->i0 = 0; p->f0 = 0; p->pad = 0; }
    __device__ __forceinline__ void load(const Packed* p) { n = p->d0; mean = p->d1; m2 = p->d2; kf = 0.0f; c = 0u; }
};

// Extremum with the reference's rule: strict compare, first occurrence wins, NaN never wins
// (every comparison with NaN is false), -0.0 and +0.0 tie.  Positions grow along a thread's
// own scan, so the strict compare keeps the thread's first occurrence; between threads a tie
// goes to the lower position.
// ABS: the extremum of |x| (norm with p = +-inf: the reference computes abs().max() / abs().min(),
// p10/src/backend/cpu/ReductionKernels.cpp:858-872, with the same scan rule).
template <bool IS_MAX, bool ABS = false>
struct ExtAcc {
    float v;
    long long i;
    __device__ __forceinline__ void init() { v = IS_MAX ? -INFINITY : INFINITY; i = kNoIndex; }
    __device__ __forceinline__ void add(float x, long long pos) {
        if (ABS) x = fabsf(x);
        bool better = IS_MAX ? (x > v) : (x < v);
        if (better) { v = x; i = pos; }
    }
    __device__ __forceinline__ void add4(float x0, float x1, float x2, float x3, long long pos, long long step) {
        add(x0, pos); add(x1, pos + step); add(x2, pos + 2 * step); add(x3, pos + 3 * step);
    }
    __device__ __forceinline__ void finish_thread() {}
    __device__ __forceinline__ void merge(const ExtAcc& o) {
        bool better = IS_MAX ? (o.v > v) : (o.v < v);
        if (better || (o.v == v && o.i < i)) { v = o.v; i = o.i; }
    }
    __device__ __forceinline__ ExtAcc shfl_down(int d) const {
        ExtAcc r;
        r.v = __shfl_down_sync(kFull, v, d);
        r.i = __shfl_down_sync(kFull, i, d);
        return r;
    }
    __device__ __forceinline__ void store(Packed* p) const { p->d0 = 0; p->d1 = 0; p->d2 = 0; p->i0 = i; p->f0 = v; p->pad = 0; }
    __device__ __forceinline__ void load(const Packed* p) { v = p->f0; i = p->i0; }
};

// Sum of |x| (F = 0) or of x*x (F = 1) in fp64: the norms with p = 1 and p = 2.  The reference
// forms abs().pow(p).sum().pow(1/p) in float32 (ReductionKernels.cpp:858-872); here every term and
// the sum are exact to fp64 rounding and the result is rounded once.
template <int F>
struct PowSumAcc {
    double s;
    __device__ __forceinline__ void init() { s = 0.0; }
    __device__ __forceinline__ void add(float x, long long) {
        const double d = (double)x;
        if (F == 0) s += fabs(d); else s = fma(d, d, s);
    }
    __device__ __forceinline__ void add4(float x0, float x1, float x2, float x3, long long, long long) {
        add(x0, 0); add(x1, 0); add(x2, 0); add(x3, 0);
    }
    __device__ __forceinline__ void finish_thread() {}
    __device__ __forceinline__ void merge(const PowSumAcc& o) { s += o.s; }
    __device__ __forceinline__ PowSumAcc shfl_down(int d) const {
        PowSumAcc r; r.s = __shfl_down_sync(kFull, s, d); return r;
    }
    __device__ __forceinline__ void store(Packed* p) const { p->d0 = s; p->d1 = 0; p->d2 = 0; p->i0 = 0; p->f0 = 0; p->pad = 0; }
    __device__ __forceinline__ void load(const Packed* p) { s = p->d0; }
};

// Product in fp64 (the reference multiplies float32 values one after the other,
// ReductionKernels.cpp:404-438, 441-513); an empty product is 1.
struct ProdAcc {
    double p;
    __device__ __forceinline__ void init() { p = 1.0; }
    __device__ __forceinline__ void add(float x, long long) { p *= (double)x; }
    __device__ __forceinline__ void add4(float x0, float x1, float x2, float x3, long long, long long) {
        p *= ((double)x0 * (double)x1) * ((double)x2 * (double)x3);
    }
    __device__ __forceinline__ void finish_thread() {}
    __device__ __forceinline__ void merge(const ProdAcc& o) { p *= o.p; }
    __device__ __forceinline__ ProdAcc shfl_down(int d) const {
        ProdAcc r; r.p = __shfl_down_sync(kFull, p, d); return r;
    }
    __device__ __forceinline__ void store(Packed* q) const { q->d0 = p; q->d1 = 0; q->d2 = 0; q->i0 = 0; q->f0 = 0; q->pad = 0; }
    __device__ __forceinline__ void load(const Packed* q) { p = q->d0; }
};

// all / any: an element counts as true iff it is not zero (static_cast<bool>, so NaN is true:
// ReductionKernels.cpp:517-563, 565-677); all of nothing is true, any of nothing is false.
template <bool IS_ALL>
struct BoolAcc {
    unsigned f;
    __device__ __forceinline__ void init() { f = IS_ALL ? 1u : 0u; }
    __device__ __forceinline__ void add(float x, long long) {
        const unsigned nz = x != 0.0f ? 1u : 0u;
        f = IS_ALL ? (f & nz) : (f | nz);
    }
    __device__ __forceinline__ void add4(float x0, float x1, float x2, float x3, long long, long long) {
        add(x0, 0); add(x1, 0); add(x2, 0); add(x3, 0);
    }
    __device__ __forceinline__ void finish_thread() {}
    __device__ __forceinline__ void merge(const BoolAcc& o) { f = IS_ALL ? (f & o.f) : (f | o.f); }
    __device__ __forceinline__ BoolAcc shfl_down(int d) const {
        BoolAcc r; r.f = __shfl_down_sync(kFull, f, d); return r;
    }
    __device__ __forceinline__ void store(Packed* p) const { p->d0 = 0; p->d1 = 0; p->d2 = 0; p->i0 = (long long)f; p->f0 = 0; p->pad = 0; }
    __device__ __forceinline__ void load(const Packed* p) { f = (unsigned)p->i0; }
};

// Fixed-order tree over the 32 lanes; lane 0 holds the result.
template <class Acc>
__device__ __forceinline__ void warp_combine(Acc& a) {
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
        Acc o = a.shfl_down(d);
        a.merge(o);
    }
}

// Fixed-order combine over a CTA (blockDim.x threads, multiple of 32, <= 1024); thread 0 holds
// the result.  `smem` must hold one Acc per warp.
template <class Acc>
__device__ __forceinline__ void block_combine(Acc& a, Acc* smem) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    warp_combine(a);
    if (nwarp == 1) return;
    if (lane == 0) smem[warp] = a;
    __syncthreads();
    if (warp == 0) {
        if (lane < nwarp) a = smem[lane]; else a.init();
        warp_combine(a);
    }
}

// ------------------------------------------------------------------ epilogues --------------
// What is written for one finished reduction.  `count` is the number of reduced elements.
struct Epilogue {
    int op;               // TPB200_OP_*
    long long correction; // var/std
};

__device__ __forceinline__ void write_result(const SumAcc& a, const Epilogue& e, double count, float* ov, long long*, long long o) {
    // mean of an empty reduction is 0/0 = NaN, as in the reference (sum 0 divided by count 0)
    *TPB_CK(&ov[o]) = e.op == TPB200_OP_MEAN ? (float)(a.s / count) : (float)a.s;
}
__device__ __forceinline__ void write_result(const MomAcc& a, const Epilogue& e, double count, float* ov, long long*, long long o) {
    // divisor max(0, n - correction), division in double, one rounding to float
    // (p10/src/backend/cpu/ReductionKernels.cpp:824-825, 844-846); an empty tensor gives NaN (:817)
    double dv = count - (double)e.correction;
    if (dv < 0.0) dv = 0.0;
    float var = count == 0.0 ? NAN : (float)(a.m2 / dv);
    *TPB_CK(&ov[o]) = e.op == TPB200_OP_STD ? sqrtf(var) : var;
}
template <int F>
__device__ __forceinline__ void write_result(const PowSumAcc<F>& a, const Epilogue&, double, float* ov, long long*, long long o) {
    *TPB_CK(&ov[o]) = F == 0 ? (float)a.s : (float)sqrt(a.s);
}
__device__ __forceinline__ void write_result(const ProdAcc& a, const Epilogue&, double, float* ov, long long*, long long o) {
    *TPB_CK(&ov[o]) = (float)a.p;
}
template <bool IS_ALL>
__device__ __forceinline__ void write_result(const BoolAcc<IS_ALL>& a, const Epilogue&, double, float* ov, long long*, long long o) {
    *TPB_CK(&reinterpret_cast<unsigned char*>(ov)[o]) = (unsigned char)a.f;   // Bool output: one byte per element
}
template <bool IS_MAX, bool ABS>
__device__ __forceinline__ void write_result(const ExtAcc<IS_MAX, ABS>& a, const Epilogue& e, double, float* ov, long long* oi, long long o) {
    // nothing compared better (empty, all NaN, or all equal to the start value): index 0 and the
    // start value, as in the reference's scan (ReductionKernels.cpp:692-694, 727-735)
    if (ov) *TPB_CK(&ov[o]) = a.v;
    if (oi) *TPB_CK(&oi[o]) = a.i == kNoIndex ? 0 : a.i;
    (void)e;
}

// ------------------------------------------------------------------ contiguous scan --------
// Feed `len` contiguous floats at p (any alignment) to acc, split over `nthr` threads with
// 128-bit loads on the 16-byte aligned body.  `pos0` is the position of p[0] in the reduction's
// row-major index space.  Each thread sees its elements in ascending position.
template <int UNROLL, class Acc>
__device__ __forceinline__ void scan_contig(Acc& acc, const float* __restrict__ p, long long len,
                                            long long pos0, int tid, int nthr) {
    // scalar head up to the first 16-byte boundary
    long long head = (long long)((4 - (((uintptr_t)p >> 2) & 3)) & 3);
    if (head > len) head = len;
    for (long long h = tid; h < head; h += nthr) acc.add(ld_stream1(p + h), pos0 + h);
    const float* q = p + head;
    const long long nvec = (len - head) >> 2;
    const long long qpos = pos0 + head;
    long long i = tid;
    const long long step = (long long)nthr * UNROLL;
    // full groups of UNROLL vectors: issue every load before the first use
    for (; i + (long long)(UNROLL - 1) * nthr < nvec; i += step) {
        float4 v[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) v[u] = ld_stream4(q + ((i + (long long)u * nthr) << 2));
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            long long b = qpos + ((i + (long long)u * nthr) << 2);
            acc.add4(v[u].x, v[u].y, v[u].z, v[u].w, b, 1);
        }
    }
    for (; i < nvec; i += nthr) {
        float4 v = ld_stream4(q + (i << 2));
        long long b = qpos + (i << 2);
        acc.add4(v.x, v.y, v.z, v.w, b, 1);
    }
    const long long done = head + (nvec << 2);
    const long long tail = len - done;
    for (long long h = tid; h < tail; h += nthr) acc.add(ld_stream1(p + done + h), pos0 + done + h);
}

}  // namespace tpb
