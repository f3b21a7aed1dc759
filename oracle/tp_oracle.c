/* TEST INFRASTRUCTURE ONLY -- a CPU restatement used as the checker in tests/, in the smoke
 * test and as the timed CPU baseline.  Nothing on the product path may call into this file.
 *
 * Plain-C restatement of TensorPlay's CPU reduction operators for float32 tensors
 * (p10/src/backend/cpu/ReductionKernels.cpp) and of the top-k contract this library defines.
 * The arithmetic ORDER and PRECISION of every step follows the reference, so results are
 * bit-identical to it (checked against the reference's own compiled code and against the
 * known answers in the reference's tests, see tests/test_oracle.py):
 *
 *   sum()            double accumulator over the logical row-major order, rounded once to float
 *                    (ReductionKernels.cpp:27-35, 72-106)
 *   sum(dims)        float output pre-filled with 0; walk ALL input indices in row-major order,
 *                    out[o] += in[i] in float (ReductionKernels.cpp:108-189, accumulate at :168)
 *   mean             the sum above divided, in float, by (float)count
 *                    (ReductionKernels.cpp:191-211; operator/(Scalar) p10/src/Tensor.cpp:446-449)
 *   max/min          running value from -inf/+inf with a STRICT compare, so the first occurrence
 *                    wins and NaN is never selected (ReductionKernels.cpp:227-315, 317-401)
 *   argmax/argmin    same scan, index of the first extremum, 0 when nothing compares greater
 *                    (ReductionKernels.cpp:682-746, 748-812)
 *   var(dims,corr)   mean(dims) in float; diff = x - mean in float; sq = diff*diff in float;
 *                    sum of sq with the sum rule above (double accumulator for the whole-tensor
 *                    overload, float sequential for the dim overload); divide in DOUBLE by
 *                    max(0, n - corr); round to float (ReductionKernels.cpp:815-847)
 *   std              sqrtf(var) (ReductionKernels.cpp:849-855)
 *   prod()           float accumulator from 1, multiplied element by element in row-major order
 *                    (ReductionKernels.cpp:404-438); prod(dims): float output pre-filled with 1,
 *                    out[o] *= in[i] over all input indices in row-major order (:441-513)
 *   norm(p)          abs() in float; pow(p) evaluated in double and stored as float
 *                    (pow_scalar_kernel, p10/src/backend/cpu/PointwiseKernels.cpp:392-396); the sum
 *                    rule above; pow(1/p) the same way (ReductionKernels.cpp:858-872);
 *                    p = +-inf: abs() then the max / min rule above
 *   all/any          an element is true iff it is not zero, so NaN is true; all of nothing is
 *                    true, any of nothing is false (ReductionKernels.cpp:517-563, 565-677)
 *
 * One deliberate difference: for argmax/argmin over a dim that is neither the last nor the
 * second-to-last of a >=3-D tensor the reference's CPU code writes its rows in a permuted order
 * (it swaps, rather than moves, the dim to the end: ReductionKernels.cpp:714-735).  This file
 * returns the mathematically meant result (first extremum along that dim, output laid out over
 * the kept dims in order), which is also what the reference's CUDA code computes.
 *
 * top-k: PARITY UNPINNED.  top-k is absent from the reference (no schema entry, kernel, binding, test
 * or golden vector), so nothing of the reference can pin this part of the file: it is held only by
 * self-consistency (sort form = heap form = numpy lexsort; k = 1 = argmax / argmin, which ARE pinned).
 * softmax / log_softmax / median below are pinned like the reductions (compiled reference, fixture).
 * The contract restated here: the first k entries of the
 * row stably sorted by value (descending when `largest`, else ascending), ties in ascending
 * index; -0.0 and +0.0 tie; NaN ranks after every number for both directions.  This follows the
 * only tie evidence in the reference, argmax/argmin's strict-compare scan (:727-735, :793-801),
 * so top-k with k = 1 equals argmax/argmin.
 *
 * Build: see oracle/Makefile (-O2 -ffp-contract=off: no fused multiply-add may merge steps the
 * reference performs as separate float operations).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define TPO_MAX_DIMS 16

enum { TPO_SUM = 0, TPO_MEAN = 1, TPO_VAR = 2, TPO_STD = 3, TPO_MAX = 4, TPO_MIN = 5,
       TPO_ARGMAX = 6, TPO_ARGMIN = 7, TPO_PROD = 8, TPO_NORM = 9, TPO_ALL = 10, TPO_ANY = 11 };

typedef struct {
    int ndim;
    int64_t size[TPO_MAX_DIMS];
    int64_t istride[TPO_MAX_DIMS];
    int64_t ostride[TPO_MAX_DIMS]; /* 0 on reduced dims */
    int64_t numel, out_numel, count;
} walk_t;

static int setup(walk_t* w, int ndim, const int64_t* sizes, const int64_t* strides, int n_dims,
                 const int64_t* dims) {
    int reduced[TPO_MAX_DIMS] = {0};
    if (ndim > TPO_MAX_DIMS) return -1;
    w->ndim = ndim;
    if (n_dims <= 0) {
        for (int i = 0; i < ndim; ++i) reduced[i] = 1;
    } else {
        for (int j = 0; j < n_dims; ++j) {
            int64_t d = dims[j];
            if (d < 0) d += ndim;
            if (d < 0 || d >= ndim) return -2; /* "Dimension out of range" */
            reduced[d] = 1;
        }
    }
    int64_t s = 1;
    for (int i = ndim - 1; i >= 0; --i) {
        w->size[i] = sizes[i];
        w->istride[i] = strides ? strides[i] : s;
        s *= sizes[i];
    }
    w->numel = s;
    int64_t os = 1, cnt = 1;
    for (int i = ndim - 1; i >= 0; --i) {
        if (reduced[i]) { w->ostride[i] = 0; cnt *= sizes[i]; }
        else { w->ostride[i] = os; os *= sizes[i]; }
    }
    w->out_numel = os;
    w->count = cnt;
    return 0;
}

/* Row-major odometer over all input indices. */
#define WALK_BEGIN(w)                                                                   \
    {                                                                                   \
        int64_t idx_[TPO_MAX_DIMS] = {0};                                               \
        int64_t ioff = 0, ooff = 0;                                                     \
        for (int64_t lin_ = 0; lin_ < (w)->numel; ++lin_) {
#define WALK_END(w)                                                                     \
            for (int d_ = (w)->ndim - 1; d_ >= 0; --d_) {                               \
                ++idx_[d_]; ioff += (w)->istride[d_]; ooff += (w)->ostride[d_];         \
                if (idx_[d_] < (w)->size[d_]) break;                                    \
                ioff -= idx_[d_] * (w)->istride[d_]; ooff -= idx_[d_] * (w)->ostride[d_]; \
                idx_[d_] = 0;                                                           \
            }                                                                           \
        }                                                                               \
    }

static float sum_full(const walk_t* w, const float* in) {
    double acc = 0.0;
    WALK_BEGIN(w) acc += (double)in[ioff]; (void)ooff; WALK_END(w)
    return (float)acc;
}

static void sum_dims(const walk_t* w, const float* in, float* out) {
    for (int64_t i = 0; i < w->out_numel; ++i) out[i] = 0.0f;
    WALK_BEGIN(w) out[ooff] += in[ioff]; WALK_END(w)
}

/* Output element count for (sizes, dims); negative on a bad dim. */
int64_t tpo_out_numel(int ndim, const int64_t* sizes, int n_dims, const int64_t* dims) {
    walk_t w;
    int rc = setup(&w, ndim, sizes, NULL, n_dims, dims);
    return rc ? rc : w.out_numel;
}

/* n_dims < 0: the overload without a dim argument.  n_dims == 0: the dim overload called with
 * an empty list, which the reference forwards to the whole-tensor kernel for sum/max/min; mean
 * then divides by the product over an empty list, i.e. by 1 (ReductionKernels.cpp:198-211).
 * Returns 0, or -2 for a bad dim, -3 for max/min of an empty tensor. */
int tpo_reduce(int op, const float* in, int ndim, const int64_t* sizes, const int64_t* strides,
               int n_dims, const int64_t* dims, int64_t correction, float* out_val,
               int64_t* out_idx) {
    walk_t w;
    int rc = setup(&w, ndim, sizes, strides, n_dims, dims);
    if (rc) return rc;
    const int full = n_dims <= 0;

    switch (op) {
    case TPO_SUM:
        if (full) out_val[0] = sum_full(&w, in);
        else sum_dims(&w, in, out_val);
        return 0;
    case TPO_MEAN: {
        if (full) {
            float cnt = n_dims < 0 ? (float)w.numel : 1.0f;
            out_val[0] = sum_full(&w, in) / cnt;
        } else {
            sum_dims(&w, in, out_val);
            float cnt = (float)w.count;
            for (int64_t i = 0; i < w.out_numel; ++i) out_val[i] = out_val[i] / cnt;
        }
        return 0;
    }
    case TPO_VAR:
    case TPO_STD: {
        if (w.numel == 0) {
            for (int64_t i = 0; i < w.out_numel; ++i) out_val[i] = NAN;
            return 0;
        }
        int64_t n = n_dims == 0 ? 1 : w.count;
        double dv = (double)(n - correction);
        if (dv < 0.0) dv = 0.0;
        if (n_dims < 0) {
            float mean = sum_full(&w, in) / (float)w.numel;
            double acc = 0.0;
            WALK_BEGIN(&w)
                float d = in[ioff] - mean;
                float sq = d * d;
                acc += (double)sq;
                (void)ooff;
            WALK_END(&w)
            float ssq = (float)acc;
            out_val[0] = (float)((double)ssq / dv);
        } else {
            float* mean = (float*)malloc(sizeof(float) * (size_t)(w.out_numel ? w.out_numel : 1));
            if (!mean) return -9;
            if (n_dims == 0) {
                mean[0] = sum_full(&w, in) / 1.0f;
                out_val[0] = 0.0f;
                /* sq.sum({}) forwards to the whole-tensor kernel: double accumulator */
                double acc = 0.0;
                WALK_BEGIN(&w)
                    float d = in[ioff] - mean[0];
                    float sq = d * d;
                    acc += (double)sq;
                    (void)ooff;
                WALK_END(&w)
                out_val[0] = (float)acc;
            } else {
                sum_dims(&w, in, mean);
                float cnt = (float)w.count;
                for (int64_t i = 0; i < w.out_numel; ++i) mean[i] = mean[i] / cnt;
                for (int64_t i = 0; i < w.out_numel; ++i) out_val[i] = 0.0f;
                WALK_BEGIN(&w)
                    float d = in[ioff] - mean[ooff];
                    float sq = d * d;
                    out_val[ooff] += sq;
                WALK_END(&w)
            }
            for (int64_t i = 0; i < w.out_numel; ++i)
                out_val[i] = (float)((double)out_val[i] / dv);
            free(mean);
        }
        if (op == TPO_STD)
            for (int64_t i = 0; i < w.out_numel; ++i) out_val[i] = sqrtf(out_val[i]);
        return 0;
    }
    case TPO_MAX:
    case TPO_MIN: {
        if (full && w.numel == 0) return -3;
        const float init = op == TPO_MAX ? -INFINITY : INFINITY;
        for (int64_t i = 0; i < w.out_numel; ++i) out_val[i] = init;
        if (op == TPO_MAX) {
            WALK_BEGIN(&w) if (in[ioff] > out_val[ooff]) out_val[ooff] = in[ioff]; WALK_END(&w)
        } else {
            WALK_BEGIN(&w) if (in[ioff] < out_val[ooff]) out_val[ooff] = in[ioff]; WALK_END(&w)
        }
        return 0;
    }
    case TPO_ARGMAX:
    case TPO_ARGMIN: {
        /* flat (n_dims < 0) or exactly one dim */
        if (n_dims == 0 || n_dims > 1) return -4;
        const float init = op == TPO_ARGMAX ? -INFINITY : INFINITY;
        float* best = (float*)malloc(sizeof(float) * (size_t)(w.out_numel ? w.out_numel : 1));
        if (!best) return -9;
        for (int64_t i = 0; i < w.out_numel; ++i) { best[i] = init; out_idx[i] = 0; }
        int rd = -1;
        if (n_dims == 1) { rd = (int)dims[0]; if (rd < 0) rd += ndim; }
        WALK_BEGIN(&w)
            float v = in[ioff];
            int better = op == TPO_ARGMAX ? (v > best[ooff]) : (v < best[ooff]);
            if (better) { best[ooff] = v; out_idx[ooff] = rd < 0 ? lin_ : idx_[rd]; }
        WALK_END(&w)
        free(best);
        return 0;
    }
    default:
        return -5;
    }
}


/* prod, norm(p), all, any.  Same dim conventions as tpo_reduce.  prod and norm write floats to
 * out; all and any write one byte (0/1) per output element to out.  Returns 0, -2 for a bad dim,
 * -3 for norm(+-inf) of an empty tensor without a dim list. */
int tpo_reduce_more(int op, const float* in, int ndim, const int64_t* sizes, const int64_t* strides,
                    int n_dims, const int64_t* dims, double p, void* out) {
    walk_t w;
    int rc = setup(&w, ndim, sizes, strides, n_dims, dims);
    if (rc) return rc;
    const int full = n_dims <= 0;
    float* of = (float*)out;
    uint8_t* ob = (uint8_t*)out;
    switch (op) {
    case TPO_PROD:
        if (full) {
            float acc = 1.0f;
            WALK_BEGIN(&w) acc *= in[ioff]; (void)ooff; WALK_END(&w)
            of[0] = acc;
        } else {
            for (int64_t i = 0; i < w.out_numel; ++i) of[i] = 1.0f;
            WALK_BEGIN(&w) of[ooff] *= in[ioff]; WALK_END(&w)
        }
        return 0;
    case TPO_NORM:
        if (isinf(p)) {
            if (full && w.numel == 0) return -3;
            const float init = p > 0 ? -INFINITY : INFINITY;
            for (int64_t i = 0; i < w.out_numel; ++i) of[i] = init;
            if (p > 0) {
                WALK_BEGIN(&w) { float a = fabsf(in[ioff]); if (a > of[ooff]) of[ooff] = a; } WALK_END(&w)
            } else {
                WALK_BEGIN(&w) { float a = fabsf(in[ioff]); if (a < of[ooff]) of[ooff] = a; } WALK_END(&w)
            }
            return 0;
        }
        if (full) {
            double acc = 0.0;
            WALK_BEGIN(&w) { float t = (float)pow((double)fabsf(in[ioff]), p); acc += (double)t; (void)ooff; } WALK_END(&w)
            of[0] = (float)pow((double)(float)acc, 1.0 / p);
        } else {
            for (int64_t i = 0; i < w.out_numel; ++i) of[i] = 0.0f;
            WALK_BEGIN(&w) { float t = (float)pow((double)fabsf(in[ioff]), p); of[ooff] += t; } WALK_END(&w)
            for (int64_t i = 0; i < w.out_numel; ++i) of[i] = (float)pow((double)of[i], 1.0 / p);
        }
        return 0;
    case TPO_ALL:
        for (int64_t i = 0; i < w.out_numel; ++i) ob[i] = 1;
        WALK_BEGIN(&w) if (!(in[ioff] != 0.0f)) ob[ooff] = 0; WALK_END(&w)
        return 0;
    case TPO_ANY:
        for (int64_t i = 0; i < w.out_numel; ++i) ob[i] = 0;
        WALK_BEGIN(&w) if (in[ioff] != 0.0f) ob[ooff] = 1; WALK_END(&w)
        return 0;
    default:
        return -5;
    }
}

/* ------------------------------------------------------------------ top-k ---------------- */

/* Rank key: larger = earlier in the output.  NaN -> 0 (after every number); -0.0 == +0.0. */
static inline uint32_t rank_key(float x, int largest) {
    uint32_t b;
    if (x != x) return 0u;
    if (x == 0.0f) x = 0.0f; /* drops the sign of -0.0 */
    memcpy(&b, &x, 4);
    b = (b & 0x80000000u) ? ~b : (b | 0x80000000u); /* ascending order-preserving */
    return largest ? b : ~b;
}

typedef struct { uint32_t key; int64_t idx; } cand_t;

/* a ranks before b */
static inline int before(cand_t a, cand_t b) {
    return a.key > b.key || (a.key == b.key && a.idx < b.idx);
}

static void merge_sort(cand_t* a, cand_t* tmp, int64_t n) {
    if (n < 2) return;
    int64_t h = n / 2;
    merge_sort(a, tmp, h);
    merge_sort(a + h, tmp, n - h);
    int64_t i = 0, j = h, o = 0;
    while (i < h && j < n) tmp[o++] = before(a[j], a[i]) ? a[j++] : a[i++];
    while (i < h) tmp[o++] = a[i++];
    while (j < n) tmp[o++] = a[j++];
    memcpy(a, tmp, sizeof(cand_t) * (size_t)n);
}

/* Definition form: full stable sort of every row.  in is [rows, len] with the given row and
 * element strides (in elements); outputs are [rows, k] contiguous. */
int tpo_topk_sort(const float* in, int64_t rows, int64_t len, int64_t row_stride,
                  int64_t elem_stride, int64_t k, int largest, float* out_val, int64_t* out_idx) {
    if (k < 0 || k > len) return -6;
    cand_t* a = (cand_t*)malloc(sizeof(cand_t) * (size_t)(len ? len : 1) * 2);
    if (!a) return -9;
    for (int64_t r = 0; r < rows; ++r) {
        const float* row = in + r * row_stride;
        for (int64_t j = 0; j < len; ++j) {
            a[j].key = rank_key(row[j * elem_stride], largest);
            a[j].idx = j;
        }
        merge_sort(a, a + len, len);
        for (int64_t j = 0; j < k; ++j) {
            out_val[r * k + j] = row[a[j].idx * elem_stride];
            out_idx[r * k + j] = a[j].idx;
        }
    }
    free(a);
    return 0;
}

static void sift_down(cand_t* h, int64_t n, int64_t i) {
    /* heap whose root is the candidate that ranks LAST among the k kept */
    for (;;) {
        int64_t l = 2 * i + 1, r = l + 1, m = i;
        if (l < n && before(h[m], h[l])) m = l;
        if (r < n && before(h[m], h[r])) m = r;
        if (m == i) return;
        cand_t t = h[i]; h[i] = h[m]; h[m] = t;
        i = m;
    }
}

/* Selection form (what a CPU implementation would run): one scan keeping the k best in a heap,
 * then a sort of the k survivors.  Same results as tpo_topk_sort. */
int tpo_topk(const float* in, int64_t rows, int64_t len, int64_t row_stride, int64_t elem_stride,
             int64_t k, int largest, float* out_val, int64_t* out_idx) {
    if (k < 0 || k > len) return -6;
    if (k == 0) return 0;
    cand_t* h = (cand_t*)malloc(sizeof(cand_t) * (size_t)k * 2);
    if (!h) return -9;
    for (int64_t r = 0; r < rows; ++r) {
        const float* row = in + r * row_stride;
        int64_t n = 0;
        for (int64_t j = 0; j < len; ++j) {
            cand_t c;
            c.key = rank_key(row[j * elem_stride], largest);
            c.idx = j;
            if (n < k) {
                h[n++] = c;
                if (n == k) for (int64_t i = k / 2 - 1; i >= 0; --i) sift_down(h, k, i);
            } else if (before(c, h[0])) {
                h[0] = c;
                sift_down(h, k, 0);
            }
        }
        merge_sort(h, h + k, k);
        for (int64_t j = 0; j < k; ++j) {
            out_val[r * k + j] = row[h[j].idx * elem_stride];
            out_idx[r * k + j] = h[j].idx;
        }
    }
    free(h);
    return 0;
}


/* ---------------------------------------------------------------- softmax / log_softmax -------
 * p10/src/backend/cpu/PointwiseKernels.cpp:519-546, step by step in float32:
 *   max_val = input.max({dim}, true)     strict-compare scan from -inf (NaN never wins)
 *   shifted = input - max_val
 *   exp_val = shifted.exp()              expf
 *   sum_exp = exp_val.sum({dim}, true)   sequential float32 accumulation along the dim
 *   softmax = exp_val / sum_exp          log_softmax = shifted - log(sum_exp)
 * in is contiguous [outer, C, inner]; out has the same layout. */
int tpo_softmax(int log, const float* in, int64_t outer, int64_t C, int64_t inner, float* out) {
    if (outer < 0 || C < 0 || inner < 0) return -1;
    for (int64_t o = 0; o < outer; ++o) {
        for (int64_t i = 0; i < inner; ++i) {
            const float* p = in + o * C * inner + i;
            float* q = out + o * C * inner + i;
            float m = -INFINITY;
            for (int64_t j = 0; j < C; ++j) {
                const float x = p[j * inner];
                if (x > m) m = x;
            }
            float s = 0.0f;
            for (int64_t j = 0; j < C; ++j) {
                const float e = expf(p[j * inner] - m);
                q[j * inner] = e;
                s += e;
            }
            if (log) {
                const float ls = logf(s);
                for (int64_t j = 0; j < C; ++j) q[j * inner] = (p[j * inner] - m) - ls;
            } else {
                for (int64_t j = 0; j < C; ++j) q[j * inner] = q[j * inner] / s;
            }
        }
    }
    return 0;
}

/* ---------------------------------------------------------------- median ----------------------
 * p10/src/backend/cpu/ReductionKernels.cpp:874-901: element (n - 1) / 2 of the sorted values (the
 * lower middle one for even n), NaN for an empty tensor.  The reference's std::nth_element leaves
 * the place of NaNs undefined; here they rank after every number. */
static int cmp_float_nan_last(const void* a, const void* b) {
    const float x = *(const float*)a, y = *(const float*)b;
    const int xn = x != x, yn = y != y;
    if (xn || yn) return xn - yn;
    return (x > y) - (x < y);
}
int tpo_median(const float* in, int64_t n, float* out) {
    if (n < 0) return -1;
    if (n == 0) { *out = NAN; return 0; }
    float* t = (float*)malloc(sizeof(float) * (size_t)n);
    if (!t) return -9;
    memcpy(t, in, sizeof(float) * (size_t)n);
    qsort(t, (size_t)n, sizeof(float), cmp_float_nan_last);
    *out = t[(n - 1) / 2];
    free(t);
    return 0;
}
