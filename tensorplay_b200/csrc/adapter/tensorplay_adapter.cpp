// Layer 2 of the drop-in: TensorPlay kernels with the exact signatures its DispatchStub casts to
// (tools/codegen/gen.py:39-54; call site p10/include/Dispatcher.h:46-59), registered for
// DispatchKey::CUDA under the operator names of p10/src/backend/cuda/ReductionKernels.cu:385-418.
// Registration is "last one wins" (p10/src/Dispatcher.cpp:13), so loading this library after
// TensorPlay replaces the cuDNN-based reductions without touching the reference.
//
// Compiled against the reference's headers (p10/include + its generated TensorGenerated.h); every
// number comes from libtpb200.so through the C ABI of include/tpb200.h.  Inputs that the sm_100a
// kernels do not handle (non-float32) fall through to the kernel that was registered before.
#include "Tensor.h"
#include "Dispatcher.h"
#include "Exception.h"

#include <algorithm>
#include <atomic>
#include <cstdint>
#include <cstdlib>
#include <limits>
#include <map>
#include <mutex>
#include <optional>
#include <string>
#include <tuple>
#include <vector>

#include <cuda_runtime_api.h>

#include "../../../include/tpb200.h"

namespace {

using tensorplay::DType;
using tensorplay::Tensor;
using IntList = std::vector<int64_t>;

// Kernels that were registered for CUDA before this library was loaded (may be absent).
struct Previous {
    void* sum = nullptr; void* sum_dim = nullptr; void* mean = nullptr; void* mean_dim = nullptr;
    void* max = nullptr; void* max_dim = nullptr; void* min = nullptr; void* min_dim = nullptr;
    void* argmax = nullptr; void* argmin = nullptr;
    void* var = nullptr; void* var_dim = nullptr; void* std_ = nullptr; void* std_dim = nullptr;
    void* prod = nullptr; void* prod_dim = nullptr; void* norm = nullptr; void* norm_dim = nullptr;
    void* all = nullptr; void* all_dim = nullptr; void* any = nullptr; void* any_dim = nullptr;
    void* topk = nullptr;
    void* softmax = nullptr; void* log_softmax = nullptr; void* median = nullptr;
    void* copy_ = nullptr;
} g_prev;

void* lookup(const char* name) {
    try {
        return tensorplay::Dispatcher::singleton().getKernel(name, tensorplay::DispatchKey::CUDA);
    } catch (...) {
        return nullptr;
    }
}

[[noreturn]] void raise_last() { TP_THROW(RuntimeError, std::string(tpb200_last_error())); }

// Calls that reached the sm_100a kernels through this adapter (a diagnostic: tests use it to show that
// TensorPlay's generated methods and its autograd nodes land here).
std::atomic<long long> g_calls{0};

// ---- device memory for results and scratch --------------------------------------------------
// The reference's CUDA allocator does one cudaMalloc per tensor and one cudaFree per release
// (p10/src/backend/cuda/CUDAAllocator.cpp:70-89), each of which synchronises the device: through the
// Dispatcher a [4096,4096] row sum then takes 20 us for a 12 us kernel.  Results and scratch of this
// adapter therefore come from a small cache of device blocks, wrapped as ordinary TensorPlay storage
// (Storage(DataPtr(ptr, deleter, device), nbytes), p10/include/Storage.h:19-25): a released block goes
// back to a free list of its size class and the next call of that size takes it without touching the
// driver.  Safe because everything TensorPlay launches runs on the legacy default stream, so a block
// that is reused is reused in stream order.  TPB200_ADAPTER_POOL=0 switches the cache off (the
// reference's allocator is then used); at most kPoolLimit bytes are kept per device.
namespace pool {
constexpr size_t kPoolLimit = 1ull << 30;
struct State {
    std::mutex mu;
    std::map<std::pair<int, size_t>, std::vector<void*>> free_;
    std::map<int, size_t> cached;
};
State& state() { static State* s = new State; return *s; }   // never destroyed: blocks may outlive static teardown
bool enabled() {
    static const bool on = [] { const char* v = std::getenv("TPB200_ADAPTER_POOL"); return !(v && v[0] == '0'); }();
    return on;
}
size_t size_class(size_t n) {
    if (n <= 512) return 512;
    if (n <= (1u << 20)) { size_t c = 512; while (c < n) c <<= 1; return c; }
    return (n + (2u << 20) - 1) / (2u << 20) * (2u << 20);
}
void release(void* p, int dev, size_t cls) {
    State& s = state();
    std::lock_guard<std::mutex> lk(s.mu);
    if (s.cached[dev] + cls <= kPoolLimit) {
        s.free_[{dev, cls}].push_back(p);
        s.cached[dev] += cls;
        return;
    }
    int cur = 0;
    cudaGetDevice(&cur);
    cudaSetDevice(dev);
    cudaFree(p);
    cudaSetDevice(cur);
}
tensorplay::DataPtr allocate(size_t nbytes, const tensorplay::Device& device) {
    const int dev = device.index() < 0 ? 0 : (int)device.index();
    const size_t cls = size_class(nbytes ? nbytes : 1);
    void* p = nullptr;
    {
        State& s = state();
        std::lock_guard<std::mutex> lk(s.mu);
        auto it = s.free_.find({dev, cls});
        if (it != s.free_.end() && !it->second.empty()) {
            p = it->second.back();
            it->second.pop_back();
            s.cached[dev] -= cls;
        }
    }
    if (!p) {
        int cur = 0;
        cudaGetDevice(&cur);
        if (cur != dev) cudaSetDevice(dev);
        const cudaError_t e = cudaMalloc(&p, cls);
        if (cur != dev) cudaSetDevice(cur);
        if (e != cudaSuccess || !p) TP_THROW(RuntimeError, "CUDA Error: out of memory in the adapter's device cache");
    }
    return tensorplay::DataPtr(p, [dev, cls](void* q) { if (q) release(q, dev, cls); }, device);
}
}  // namespace pool

// A fresh tensor on `device`: from the cache above, or through the reference's allocator.
Tensor fresh(const IntList& shape, DType dtype, const tensorplay::Device& device) {
    if (!pool::enabled()) return Tensor(shape, dtype, device);
    size_t numel = 1;
    for (int64_t v : shape) numel *= (size_t)v;
    const size_t item = dtype == DType::Int64 ? 8 : (dtype == DType::Float32 ? 4 : 1);   // the dtypes this adapter makes
    const size_t nbytes = numel * item;
    tensorplay::Storage st(pool::allocate(nbytes, device), nbytes);
    return Tensor(st, shape, dtype);
}

// (mask, output shape) for a dim list; an empty list reduces every dim.  Errors as
// compute_reduction_shape (p10/src/backend/cpu/ReductionKernels.cpp:48-58).
uint64_t mask_and_shape(const Tensor& self, const IntList& dims, bool keepdim, IntList* out_shape) {
    const int64_t nd = self.dim();
    uint64_t mask = 0;
    for (int64_t d : dims) {
        if (d < 0) d += nd;
        if (d < 0 || d >= nd) TP_THROW(RuntimeError, "Dimension out of range");
        mask |= 1ull << d;
    }
    const bool all = dims.empty();
    const IntList shape = static_cast<IntList>(self.shape());
    for (int64_t i = 0; i < nd; ++i) {
        const bool red = all || ((mask >> i) & 1);
        if (red) { if (keepdim && !all) out_shape->push_back(1); }
        else out_shape->push_back(shape[i]);
    }
    return all ? 0 : mask;
}

// One reduction through the C ABI on the legacy default stream (where the reference launches:
// ReductionKernels.cu:86-95).  Results and scratch are ordinary TensorPlay tensors.
Tensor run(int op, const Tensor& self, uint64_t mask, int index_dim, int64_t correction, const IntList& out_shape) {
    const int nd = (int)self.dim();
    const IntList sizes = static_cast<IntList>(self.shape());
    const IntList strides = self.strides();
    const bool idx = op == TPB200_OP_ARGMAX || op == TPB200_OP_ARGMIN;
    const bool boolean = op == TPB200_OP_ALL || op == TPB200_OP_ANY;
    Tensor out = fresh(out_shape, idx ? DType::Int64 : (boolean ? DType::Bool : DType::Float32), self.device());
    const size_t ws_bytes = tpb200_reduce_workspace_bytes(op, TPB200_F32, nd, sizes.data(), strides.data(), mask);
    Tensor ws;
    if (ws_bytes) ws = fresh(IntList{(int64_t)ws_bytes}, DType::UInt8, self.device());
    g_calls.fetch_add(1, std::memory_order_relaxed);
    const int rc = tpb200_reduce(op, self.data_ptr(), TPB200_F32, nd, sizes.data(), strides.data(), mask, index_dim,
                                 correction, idx ? nullptr : out.data_ptr(), idx ? out.data_ptr<int64_t>() : nullptr,
                                 ws_bytes ? ws.data_ptr() : nullptr, ws_bytes, nullptr);
    if (rc != TPB200_OK) raise_last();
    return out;
}

// float32 tensors of at most TPB200_MAX_DIMS dims run here; everything else goes to the kernel that
// was registered before (TPB200_ERR_UNSUPPORTED exists for exactly that)
bool ours(const Tensor& self) { return self.dtype() == DType::Float32 && self.dim() <= TPB200_MAX_DIMS; }
bool same_dtype(DType d) { return d == DType::Undefined || d == DType::Float32; }

template <class Fn, class... A>
Tensor fallthrough(void* prev, const char* name, A&&... a) {
    if (!prev) TP_THROW(NotImplementedError, std::string(name) + " not implemented for this dtype on CUDA");
    return reinterpret_cast<Fn>(prev)(std::forward<A>(a)...);
}

// ---- the kernels ------------------------------------------------------------------------------
Tensor tpb_sum(const Tensor& self, DType dtype) {
    if (!ours(self) || !same_dtype(dtype)) return fallthrough<Tensor (*)(const Tensor&, DType)>(g_prev.sum, "sum", self, dtype);
    return run(TPB200_OP_SUM, self, 0, -1, 1, {});
}
Tensor tpb_sum_dim(const Tensor& self, const IntList& dim, bool keepdim, DType dtype) {
    if (!ours(self) || !same_dtype(dtype))
        return fallthrough<Tensor (*)(const Tensor&, const IntList&, bool, DType)>(g_prev.sum_dim, "sum", self, dim, keepdim, dtype);
    IntList shape; const uint64_t m = mask_and_shape(self, dim, keepdim, &shape);
    return run(TPB200_OP_SUM, self, m, -1, 1, shape);
}
Tensor tpb_mean(const Tensor& self, DType dtype) {
    if (!ours(self) || !same_dtype(dtype)) return fallthrough<Tensor (*)(const Tensor&, DType)>(g_prev.mean, "mean", self, dtype);
    return run(TPB200_OP_MEAN, self, 0, -1, 1, {});
}
Tensor tpb_mean_dim(const Tensor& self, const IntList& dim, bool keepdim, DType dtype) {
    if (!ours(self) || !same_dtype(dtype))
        return fallthrough<Tensor (*)(const Tensor&, const IntList&, bool, DType)>(g_prev.mean_dim, "mean", self, dim, keepdim, dtype);
    IntList shape; const uint64_t m = mask_and_shape(self, dim, keepdim, &shape);
    return run(TPB200_OP_MEAN, self, m, -1, 1, shape);
}
Tensor tpb_max(const Tensor& self) {
    if (!ours(self)) return fallthrough<Tensor (*)(const Tensor&)>(g_prev.max, "max", self);
    return run(TPB200_OP_MAX, self, 0, -1, 1, {});
}
Tensor tpb_max_dim(const Tensor& self, const IntList& dim, bool keepdim) {
    if (!ours(self)) return fallthrough<Tensor (*)(const Tensor&, const IntList&, bool)>(g_prev.max_dim, "max", self, dim, keepdim);
    IntList shape; const uint64_t m = mask_and_shape(self, dim, keepdim, &shape);
    return run(TPB200_OP_MAX, self, m, -1, 1, shape);
}
Tensor tpb_min(const Tensor& self) {
    if (!ours(self)) return fallthrough<Tensor (*)(const Tensor&)>(g_prev.min, "min", self);
    return run(TPB200_OP_MIN, self, 0, -1, 1, {});
}
Tensor tpb_min_dim(const Tensor& self, const IntList& dim, bool keepdim) {
    if (!ours(self)) return fallthrough<Tensor (*)(const Tensor&, const IntList&, bool)>(g_prev.min_dim, "min", self, dim, keepdim);
    IntList shape; const uint64_t m = mask_and_shape(self, dim, keepdim, &shape);
    return run(TPB200_OP_MIN, self, m, -1, 1, shape);
}
Tensor arg_common(int op, void* prev, const char* name, const Tensor& self, std::optional<int64_t> dim, bool keepdim) {
    if (!ours(self)) return fallthrough<Tensor (*)(const Tensor&, std::optional<int64_t>, bool)>(prev, name, self, dim, keepdim);
    if (!dim.has_value()) return run(op, self, 0, -1, 1, {});
    int64_t d = *dim;
    if (d < 0) d += self.dim();
    if (d < 0 || d >= self.dim()) TP_THROW(RuntimeError, "Dimension out of range");
    IntList shape; const uint64_t m = mask_and_shape(self, IntList{d}, keepdim, &shape);
    return run(op, self, m, (int)d, 1, shape);
}
Tensor tpb_argmax(const Tensor& self, std::optional<int64_t> dim, bool keepdim) {
    return arg_common(TPB200_OP_ARGMAX, g_prev.argmax, "argmax", self, dim, keepdim);
}
Tensor tpb_argmin(const Tensor& self, std::optional<int64_t> dim, bool keepdim) {
    return arg_common(TPB200_OP_ARGMIN, g_prev.argmin, "argmin", self, dim, keepdim);
}
Tensor tpb_var(const Tensor& self, int64_t correction) {
    if (!ours(self)) return fallthrough<Tensor (*)(const Tensor&, int64_t)>(g_prev.var, "var", self, correction);
    return run(TPB200_OP_VAR, self, 0, -1, correction, {});
}
Tensor tpb_var_dim(const Tensor& self, const IntList& dim, int64_t correction, bool keepdim) {
    if (!ours(self)) return fallthrough<Tensor (*)(const Tensor&, const IntList&, int64_t, bool)>(g_prev.var_dim, "var", self, dim, correction, keepdim);
    IntList shape; const uint64_t m = mask_and_shape(self, dim, keepdim, &shape);
    return run(TPB200_OP_VAR, self, m, -1, correction, shape);
}
Tensor tpb_std(const Tensor& self, int64_t correction) {
    if (!ours(self)) return fallthrough<Tensor (*)(const Tensor&, int64_t)>(g_prev.std_, "std", self, correction);
    return run(TPB200_OP_STD, self, 0, -1, correction, {});
}
Tensor tpb_std_dim(const Tensor& self, const IntList& dim, int64_t correction, bool keepdim) {
    if (!ours(self)) return fallthrough<Tensor (*)(const Tensor&, const IntList&, int64_t, bool)>(g_prev.std_dim, "std", self, dim, correction, keepdim);
    IntList shape; const uint64_t m = mask_and_shape(self, dim, keepdim, &shape);
    return run(TPB200_OP_STD, self, m, -1, correction, shape);
}

Tensor tpb_prod(const Tensor& self, DType dtype) {
    if (!ours(self) || !same_dtype(dtype)) return fallthrough<Tensor (*)(const Tensor&, DType)>(g_prev.prod, "prod", self, dtype);
    return run(TPB200_OP_PROD, self, 0, -1, 1, {});
}
Tensor tpb_prod_dim(const Tensor& self, const IntList& dim, bool keepdim, DType dtype) {
    if (!ours(self) || !same_dtype(dtype))
        return fallthrough<Tensor (*)(const Tensor&, const IntList&, bool, DType)>(g_prev.prod_dim, "prod", self, dim, keepdim, dtype);
    IntList shape; const uint64_t m = mask_and_shape(self, dim, keepdim, &shape);
    return run(TPB200_OP_PROD, self, m, -1, 1, shape);
}
// p = 1, 2, +-inf run here; any other p goes to the kernel registered before (the reference's own
// CUDA kernel rejects everything but p = 2: ReductionKernels.cu:296-321)
int norm_op(double p) {
    if (p == 1.0) return TPB200_OP_NORM1;
    if (p == 2.0) return TPB200_OP_NORM2;
    if (p == std::numeric_limits<double>::infinity()) return TPB200_OP_NORM_INF;
    if (p == -std::numeric_limits<double>::infinity()) return TPB200_OP_NORM_NEG_INF;
    return -1;
}
Tensor tpb_norm(const Tensor& self, double p) {
    const int op = norm_op(p);
    if (!ours(self) || op < 0) return fallthrough<Tensor (*)(const Tensor&, double)>(g_prev.norm, "norm", self, p);
    return run(op, self, 0, -1, 1, {});
}
Tensor tpb_norm_dim(const Tensor& self, const IntList& dim, double p, bool keepdim) {
    const int op = norm_op(p);
    if (!ours(self) || op < 0)
        return fallthrough<Tensor (*)(const Tensor&, const IntList&, double, bool)>(g_prev.norm_dim, "norm", self, dim, p, keepdim);
    IntList shape; const uint64_t m = mask_and_shape(self, dim, keepdim, &shape);
    return run(op, self, m, -1, 1, shape);
}
Tensor tpb_all(const Tensor& self) {
    if (!ours(self)) return fallthrough<Tensor (*)(const Tensor&)>(g_prev.all, "all", self);
    return run(TPB200_OP_ALL, self, 0, -1, 1, {});
}
Tensor tpb_all_dim(const Tensor& self, const IntList& dim, bool keepdim) {
    if (!ours(self)) return fallthrough<Tensor (*)(const Tensor&, const IntList&, bool)>(g_prev.all_dim, "all", self, dim, keepdim);
    IntList shape; const uint64_t m = mask_and_shape(self, dim, keepdim, &shape);
    return run(TPB200_OP_ALL, self, m, -1, 1, shape);
}
Tensor tpb_any(const Tensor& self) {
    if (!ours(self)) return fallthrough<Tensor (*)(const Tensor&)>(g_prev.any, "any", self);
    return run(TPB200_OP_ANY, self, 0, -1, 1, {});
}
Tensor tpb_any_dim(const Tensor& self, const IntList& dim, bool keepdim) {
    if (!ours(self)) return fallthrough<Tensor (*)(const Tensor&, const IntList&, bool)>(g_prev.any_dim, "any", self, dim, keepdim);
    IntList shape; const uint64_t m = mask_and_shape(self, dim, keepdim, &shape);
    return run(TPB200_OP_ANY, self, m, -1, 1, shape);
}

// topk(Tensor self, int64_t k, int64_t dim=-1, bool largest=true, bool sorted=true) -> (values, indices):
// a new operator (schema entry: topk_schema.yaml beside this file; the generated Tensor::topk
// reaches this function as DispatchStub<std::tuple<Tensor, Tensor>, const Tensor&, int64_t, int64_t,
// bool, bool>).  The kernels write [other dims..., k]; for dim != last the result is handed back as
// the permuted view that puts k where `dim` was.
std::tuple<Tensor, Tensor> tpb_topk(const Tensor& self, int64_t k, int64_t dim, bool largest, bool sorted) {
    using Fn = std::tuple<Tensor, Tensor> (*)(const Tensor&, int64_t, int64_t, bool, bool);
    if (!ours(self) || self.dim() > TPB200_MAX_DIMS) {
        if (!g_prev.topk) TP_THROW(NotImplementedError, "topk not implemented for this dtype on CUDA");
        return reinterpret_cast<Fn>(g_prev.topk)(self, k, dim, largest, sorted);
    }
    const int nd = (int)self.dim();
    int64_t d = dim < 0 ? dim + std::max(nd, 1) : dim;
    if (d < 0 || d >= std::max(nd, 1)) TP_THROW(RuntimeError, "Dimension out of range");
    const IntList sizes = static_cast<IntList>(self.shape());
    const IntList strides = self.strides();
    if (k < 0 || k > (nd ? sizes[d] : 1)) TP_THROW(RuntimeError, "selected index k out of range");
    IntList inner;                                   // [other dims in their order..., k]
    for (int i = 0; i < nd; ++i) if (i != d) inner.push_back(sizes[i]);
    inner.push_back(k);
    Tensor values = fresh(inner, DType::Float32, self.device());
    Tensor indices = fresh(inner, DType::Int64, self.device());
    const size_t ws_bytes = tpb200_topk_workspace_bytes(TPB200_F32, nd, sizes.data(), strides.data(), (int)d, k);
    Tensor ws;
    if (ws_bytes) ws = fresh(IntList{(int64_t)ws_bytes}, DType::UInt8, self.device());
    g_calls.fetch_add(1, std::memory_order_relaxed);
    const int rc = tpb200_topk(self.data_ptr(), TPB200_F32, nd, sizes.data(), strides.data(), (int)d, k, largest ? 1 : 0,
                               sorted ? 1 : 0, values.data_ptr(), indices.data_ptr<int64_t>(),
                               ws_bytes ? ws.data_ptr() : nullptr, ws_bytes, nullptr);
    if (rc == TPB200_ERR_UNSUPPORTED && g_prev.topk) return reinterpret_cast<Fn>(g_prev.topk)(self, k, dim, largest, sorted);
    if (rc != TPB200_OK) raise_last();
    if (nd == 0 || d == nd - 1) return {values, indices};
    // view with k moved from the last position back to `dim`
    IntList shape, vstrides;
    IntList cs(inner.size());
    int64_t acc = 1;
    for (int i = (int)inner.size() - 1; i >= 0; --i) { cs[i] = acc; acc *= inner[i]; }
    for (int i = 0, j = 0; i < nd; ++i) {
        if (i == d) { shape.push_back(k); vstrides.push_back(cs[nd - 1]); }
        else { shape.push_back(inner[j]); vstrides.push_back(cs[j]); ++j; }
    }
    return {Tensor(values.impl()->storage(), shape, vstrides, DType::Float32, 0),
            Tensor(indices.impl()->storage(), shape, vstrides, DType::Int64, 0)};
}

// softmax / log_softmax (native_functions.yaml:587-597; the reference's CUDA kernels are
// softmax_kernel_cudnn / log_softmax_kernel_cudnn, ActivationKernels.cu:172-181).  Layouts the
// kernels do not take (a non-contiguous tensor with dim != last) go to the kernel registered before.
Tensor softmax_common(int log, void* prev, const char* name, const Tensor& self, int64_t dim, DType dtype) {
    using Fn = Tensor (*)(const Tensor&, int64_t, DType);
    if (!ours(self) || !same_dtype(dtype) || self.dim() == 0) return fallthrough<Fn>(prev, name, self, dim, dtype);
    const int nd = (int)self.dim();
    int64_t d = dim < 0 ? dim + nd : dim;
    if (d < 0 || d >= nd) TP_THROW(RuntimeError, "Dimension out of range");
    const IntList sizes = static_cast<IntList>(self.shape());
    const IntList strides = self.strides();
    Tensor out = fresh(sizes, DType::Float32, self.device());
    g_calls.fetch_add(1, std::memory_order_relaxed);
    const int rc = tpb200_softmax(log, self.data_ptr(), TPB200_F32, nd, sizes.data(), strides.data(), (int)d,
                                  out.data_ptr(), nullptr);
    if (rc == TPB200_ERR_UNSUPPORTED && prev) return reinterpret_cast<Fn>(prev)(self, dim, dtype);
    if (rc != TPB200_OK) raise_last();
    return out;
}
Tensor tpb_softmax(const Tensor& self, int64_t dim, DType dtype) {
    return softmax_common(0, g_prev.softmax, "softmax", self, dim, dtype);
}
Tensor tpb_log_softmax(const Tensor& self, int64_t dim, DType dtype) {
    return softmax_common(1, g_prev.log_softmax, "log_softmax", self, dim, dtype);
}
// median(Tensor self) -> Tensor (native_functions.yaml:796-799): the reference registers a CPU kernel
// only; this gives CUDA tensors one.  Result: a 0-dim Float32 tensor on the input's device.
Tensor tpb_median(const Tensor& self) {
    if (!ours(self)) return fallthrough<Tensor (*)(const Tensor&)>(g_prev.median, "median", self);
    const int nd = (int)self.dim();
    const IntList sizes = static_cast<IntList>(self.shape());
    const IntList strides = self.strides();
    Tensor out = fresh(IntList{}, DType::Float32, self.device());
    const size_t ws_bytes = tpb200_median_workspace_bytes();
    Tensor ws = fresh(IntList{(int64_t)ws_bytes}, DType::UInt8, self.device());
    g_calls.fetch_add(1, std::memory_order_relaxed);
    const int rc = tpb200_median(self.numel() ? self.data_ptr() : nullptr, TPB200_F32, nd, sizes.data(), strides.data(),
                                 out.data_ptr(), ws.data_ptr(), ws_bytes, nullptr);
    if (rc != TPB200_OK) raise_last();
    return out;
}

// copy_(Tensor& self, const Tensor& src) (native_functions.yaml; the reference's CUDA kernel is copy_kernel,
// p10/src/backend/cuda/CopyKernels.cu:56-160).  Taken here: both tensors on the same CUDA device, the same
// 4-byte dtype, the same shape, and at least one of them not contiguous -- the strided copies that
// permute().contiguous() and friends make.  Everything else (casts, host sources, plain contiguous
// copies, which the reference does with one cudaMemcpy) goes to the kernel registered before.
Tensor& tpb_copy_(Tensor& self, const Tensor& src) {
    using Fn = Tensor& (*)(Tensor&, const Tensor&);
    const bool four = self.dtype() == src.dtype() && (self.dtype() == DType::Float32 || self.dtype() == DType::Int32 || self.dtype() == DType::UInt32);
    const bool ours_ = four && self.device().is_cuda() && src.device().is_cuda() && self.device() == src.device() &&
                       static_cast<IntList>(self.shape()) == static_cast<IntList>(src.shape()) &&
                       !(self.is_contiguous() && src.is_contiguous()) && self.dim() <= TPB200_MAX_DIMS;
    if (!ours_) {
        if (!g_prev.copy_) TP_THROW(NotImplementedError, "copy_ not implemented for these tensors on CUDA");
        return reinterpret_cast<Fn>(g_prev.copy_)(self, src);
    }
    const IntList sizes = static_cast<IntList>(self.shape());
    const IntList ds = self.strides(), ss = src.strides();
    g_calls.fetch_add(1, std::memory_order_relaxed);
    const int rc = tpb200_strided_copy(self.data_ptr(), ds.data(), src.data_ptr(), ss.data(), TPB200_F32, (int)self.dim(),
                                       sizes.data(), nullptr);
    if (rc != TPB200_OK) raise_last();
    return self;
}

}  // namespace

extern "C" long long tpb200_adapter_calls(void) { return g_calls.load(std::memory_order_relaxed); }

namespace tensorplay {

TENSORPLAY_LIBRARY_IMPL(CUDA, B200Reductions) {
    g_prev.sum = lookup("sum");         g_prev.sum_dim = lookup("sum.dim_IntList");
    g_prev.mean = lookup("mean");       g_prev.mean_dim = lookup("mean.dim");
    g_prev.max = lookup("max");         g_prev.max_dim = lookup("max.dim");
    g_prev.min = lookup("min");         g_prev.min_dim = lookup("min.dim");
    g_prev.argmax = lookup("argmax");   g_prev.argmin = lookup("argmin");
    g_prev.var = lookup("var");         g_prev.var_dim = lookup("var.dim");
    g_prev.std_ = lookup("std");        g_prev.std_dim = lookup("std.dim");
    g_prev.prod = lookup("prod");       g_prev.prod_dim = lookup("prod.dim_IntList");
    g_prev.norm = lookup("norm");       g_prev.norm_dim = lookup("norm.dim");
    g_prev.all = lookup("all");         g_prev.all_dim = lookup("all.dim");
    g_prev.any = lookup("any");         g_prev.any_dim = lookup("any.dim");
    g_prev.topk = lookup("topk");
    g_prev.softmax = lookup("softmax"); g_prev.log_softmax = lookup("log_softmax"); g_prev.median = lookup("median");
    g_prev.copy_ = lookup("copy_");
    m.impl("sum", tpb_sum);             m.impl("sum.dim_IntList", tpb_sum_dim);
    m.impl("mean", tpb_mean);           m.impl("mean.dim", tpb_mean_dim);
    m.impl("max", tpb_max);             m.impl("max.dim", tpb_max_dim);
    m.impl("min", tpb_min);             m.impl("min.dim", tpb_min_dim);
    m.impl("argmax", tpb_argmax);       m.impl("argmin", tpb_argmin);
    m.impl("var", tpb_var);             m.impl("var.dim", tpb_var_dim);
    m.impl("std", tpb_std);             m.impl("std.dim", tpb_std_dim);
    m.impl("prod", tpb_prod);           m.impl("prod.dim_IntList", tpb_prod_dim);
    m.impl("norm", tpb_norm);           m.impl("norm.dim", tpb_norm_dim);
    m.impl("all", tpb_all);             m.impl("all.dim", tpb_all_dim);
    m.impl("any", tpb_any);             m.impl("any.dim", tpb_any_dim);
    m.impl("topk", tpb_topk);
    m.impl("softmax", tpb_softmax);     m.impl("log_softmax", tpb_log_softmax);
    m.impl("median", tpb_median);
    m.impl("copy_", tpb_copy_);
}

}  // namespace tensorplay
