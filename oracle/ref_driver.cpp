// TEST INFRASTRUCTURE ONLY -- never linked into, or called from, the product path.
//
// C entry points over the *unmodified* TensorPlay CPU reduction path, so that tests and the
// CPU-baseline leg of the benchmark can run the reference's own code on raw float buffers.
// This file is compiled by oracle/build_ref.sh together with the reference's own sources
// (p10/src/*.cpp, p10/src/backend/cpu/*Kernels.cpp and the file its generator emits); it
// contains no reduction arithmetic of its own.  Every call goes through the reference's
// generated Tensor methods and therefore through its Dispatcher:
//   Tensor::sum/mean/max/min/argmax/argmin/var/std/prod/norm/all/any/softmax/log_softmax/median
//   ->  DispatchStub::call(name, CPU, ...)
//   ->  tensorplay::cpu::*_kernel   (p10/src/backend/cpu/ReductionKernels.cpp:72-872)
#include "Tensor.h"

#include <cstdint>
#include <cstring>
#include <optional>
#include <string>
#include <vector>

using namespace tensorplay;

namespace {
thread_local std::string g_err;

Tensor wrap(const float* in, int ndim, const int64_t* sizes, const int64_t* strides) {
    std::vector<int64_t> sz(sizes, sizes + ndim), st(ndim);
    int64_t span = 1;
    bool empty = false;
    if (strides) {
        for (int i = 0; i < ndim; ++i) {
            st[i] = strides[i];
            if (sz[i] == 0) empty = true;
            else span += (sz[i] - 1) * st[i];
        }
    } else {
        int64_t s = 1;
        for (int i = ndim - 1; i >= 0; --i) { st[i] = s; s *= sz[i]; }
        span = s;
        if (s == 0) empty = true;
    }
    if (empty) span = 0;
    Storage storage(DataPtr(const_cast<float*>(in), deleteNothing, Device(DeviceType::CPU)),
                    static_cast<size_t>(span) * sizeof(float));
    return Tensor(storage, sz, st, DType::Float32, 0);
}
}  // namespace

extern "C" {

const char* tpref_last_error(void) { return g_err.c_str(); }

// op: 0 sum, 1 mean, 2 var, 3 std, 4 max, 5 min, 6 argmax, 7 argmin.
// n_dims < 0 selects the overload without a dim argument (whole tensor); otherwise dims[0..n_dims)
// is passed as the reference's dim list (argmax/argmin take dims[0] only).
// Value results are written to out_val (float), index results to out_idx (int64); the caller
// sizes them from the expected output shape and passes that element count in out_numel.
int tpref_reduce(int op, const float* in, int ndim, const int64_t* sizes, const int64_t* strides,
                 int n_dims, const int64_t* dims, int keepdim, int64_t correction,
                 float* out_val, int64_t* out_idx, int64_t out_numel) {
    try {
        Tensor x = wrap(in, ndim, sizes, strides);
        std::vector<int64_t> d;
        if (n_dims > 0) d.assign(dims, dims + n_dims);
        const bool full = n_dims < 0;
        const bool kd = keepdim != 0;
        Tensor r;
        switch (op) {
            case 0: r = full ? x.sum(DType::Undefined) : x.sum(d, kd, DType::Undefined); break;
            case 1: r = full ? x.mean(DType::Undefined) : x.mean(d, kd, DType::Undefined); break;
            case 2: r = full ? x.var(correction) : x.var(d, correction, kd); break;
            case 3: r = full ? x.std(correction) : x.std(d, correction, kd); break;
            case 4: r = full ? x.max() : x.max(d, kd); break;
            case 5: r = full ? x.min() : x.min(d, kd); break;
            case 6: r = full ? x.argmax(std::nullopt, false) : x.argmax(std::optional<int64_t>(d.at(0)), kd); break;
            case 7: r = full ? x.argmin(std::nullopt, false) : x.argmin(std::optional<int64_t>(d.at(0)), kd); break;
            default: g_err = "unknown op"; return 2;
        }
        if (r.numel() != out_numel) {
            g_err = "output element count mismatch: reference produced " + std::to_string(r.numel());
            return 3;
        }
        Tensor rc = r.is_contiguous() ? r : r.clone();
        if (op >= 6) {
            if (rc.dtype() != DType::Int64) { g_err = "expected Int64 result"; return 4; }
            std::memcpy(out_idx, rc.data_ptr<int64_t>(), sizeof(int64_t) * out_numel);
        } else {
            if (rc.dtype() != DType::Float32) { g_err = "expected Float32 result"; return 4; }
            std::memcpy(out_val, rc.data_ptr<float>(), sizeof(float) * out_numel);
        }
        return 0;
    } catch (const std::exception& e) {
        g_err = e.what();
        return 1;
    }
}

// op: 8 prod, 9 norm(p), 10 all, 11 any; dim conventions as tpref_reduce.  prod and norm write
// floats to out, all and any one byte per output element.
int tpref_reduce_more(int op, const float* in, int ndim, const int64_t* sizes, const int64_t* strides,
                      int n_dims, const int64_t* dims, int keepdim, double p, void* out,
                      int64_t out_numel) {
    try {
        Tensor x = wrap(in, ndim, sizes, strides);
        std::vector<int64_t> d;
        if (n_dims > 0) d.assign(dims, dims + n_dims);
        const bool full = n_dims < 0;
        const bool kd = keepdim != 0;
        Tensor r;
        switch (op) {
            case 8: r = full ? x.prod(DType::Undefined) : x.prod(d, kd, DType::Undefined); break;
            case 9: r = full ? x.norm(p) : x.norm(d, p, kd); break;
            case 10: r = full ? x.all() : x.all(d, kd); break;
            case 11: r = full ? x.any() : x.any(d, kd); break;
            default: g_err = "unknown op"; return 2;
        }
        if (r.numel() != out_numel) {
            g_err = "output element count mismatch: reference produced " + std::to_string(r.numel());
            return 3;
        }
        Tensor rc = r.is_contiguous() ? r : r.clone();
        if (op >= 10) {
            if (rc.dtype() != DType::Bool) { g_err = "expected Bool result"; return 4; }
            std::memcpy(out, rc.data_ptr<bool>(), sizeof(bool) * out_numel);
        } else {
            if (rc.dtype() != DType::Float32) { g_err = "expected Float32 result"; return 4; }
            std::memcpy(out, rc.data_ptr<float>(), sizeof(float) * out_numel);
        }
        return 0;
    } catch (const std::exception& e) {
        g_err = e.what();
        return 1;
    }
}

// softmax (log = 0) / log_softmax (log = 1) along `dim` through Tensor::softmax / Tensor::log_softmax
// (p10/src/backend/cpu/PointwiseKernels.cpp:519-546); out receives the result in row-major order.
int tpref_softmax(int log, const float* in, int ndim, const int64_t* sizes, const int64_t* strides,
                  int64_t dim, float* out, int64_t out_numel) {
    try {
        Tensor x = wrap(in, ndim, sizes, strides);
        Tensor r = log ? x.log_softmax(dim, DType::Undefined) : x.softmax(dim, DType::Undefined);
        if (r.numel() != out_numel) { g_err = "output element count mismatch"; return 3; }
        Tensor rc = r.is_contiguous() ? r : r.clone();
        if (rc.dtype() != DType::Float32) { g_err = "expected Float32 result"; return 4; }
        std::memcpy(out, rc.data_ptr<float>(), sizeof(float) * out_numel);
        return 0;
    } catch (const std::exception& e) {
        g_err = e.what();
        return 1;
    }
}

// median of the whole tensor through Tensor::median (p10/src/backend/cpu/ReductionKernels.cpp:874-901).
int tpref_median(const float* in, int ndim, const int64_t* sizes, const int64_t* strides, float* out) {
    try {
        Tensor x = wrap(in, ndim, sizes, strides);
        Tensor r = x.median();
        if (r.numel() != 1 || r.dtype() != DType::Float32) { g_err = "expected one Float32 value"; return 4; }
        *out = *r.data_ptr<float>();
        return 0;
    } catch (const std::exception& e) {
        g_err = e.what();
        return 1;
    }
}

}  // extern "C"
