// TEST INFRASTRUCTURE.  Exercises the drop-in boundary end to end at the C++ level: TensorPlay's own
// generated Tensor methods, called on CUDA tensors, must resolve through TensorPlay's Dispatcher to
// the kernels registered by tensorplay_b200/csrc/adapter/tensorplay_adapter.cpp and agree with the
// same methods run on the CPU copy of the data (the reference's CPU kernels).
// Built by oracle/build_adapter_check.sh against a TensorPlay checkout; run by tests/test_gpu_adapter.py.
#include "Tensor.h"

#include <cuda_runtime.h>

#include <cmath>
#include <cstdio>
#include <cstring>
#include <ctime>
#include <limits>
#include <vector>

using namespace tensorplay;

// the CPU checker's top-k (oracle/tp_oracle.c): [rows, len] with strides in elements -> [rows, k]
extern "C" int tpo_topk(const float* in, int64_t rows, int64_t len, int64_t row_stride, int64_t elem_stride,
                        int64_t k, int largest, float* out_val, int64_t* out_idx);

static Tensor to_cuda(const Tensor& c) {
    Tensor g(static_cast<std::vector<int64_t>>(c.shape()), c.dtype(), Device(DeviceType::CUDA, 0));
    cudaMemcpy(g.data_ptr(), c.data_ptr(), c.numel() * c.itemsize(), cudaMemcpyHostToDevice);
    return g;
}
template <class T>
static std::vector<T> to_host(const Tensor& g) {
    std::vector<T> h(g.numel());
    cudaDeviceSynchronize();
    cudaMemcpy(h.data(), g.data_ptr(), h.size() * sizeof(T), cudaMemcpyDeviceToHost);
    return h;
}
static int fails = 0, checks = 0;
static void close_f(const char* what, const Tensor& gpu, const Tensor& cpu, double rel, double abs_tol) {
    ++checks;
    auto g = to_host<float>(gpu);
    const float* c = cpu.data_ptr<float>();
    if ((int64_t)g.size() != cpu.numel() || static_cast<std::vector<int64_t>>(gpu.shape()) != static_cast<std::vector<int64_t>>(cpu.shape())) {
        printf("FAIL %s: shape\n", what); ++fails; return;
    }
    for (size_t i = 0; i < g.size(); ++i)
        if (!(std::fabs((double)g[i] - c[i]) <= rel * std::fabs((double)c[i]) + abs_tol)) {
            printf("FAIL %s: [%zu] gpu %.9g cpu %.9g\n", what, i, g[i], c[i]); ++fails; return;
        }
}
static void equal_i(const char* what, const Tensor& gpu, const Tensor& cpu) {
    ++checks;
    auto g = to_host<int64_t>(gpu);
    const int64_t* c = cpu.data_ptr<int64_t>();
    for (size_t i = 0; i < g.size(); ++i)
        if (g[i] != c[i]) { printf("FAIL %s: [%zu] gpu %lld cpu %lld\n", what, i, (long long)g[i], (long long)c[i]); ++fails; return; }
}
static void equal_bool(const char* what, const Tensor& gpu, const Tensor& cpu) {
    ++checks;
    if (gpu.dtype() != DType::Bool) { printf("FAIL %s: not a Bool tensor\n", what); ++fails; return; }
    auto g = to_host<unsigned char>(gpu);
    const bool* c = cpu.data_ptr<bool>();
    if ((int64_t)g.size() != cpu.numel()) { printf("FAIL %s: shape\n", what); ++fails; return; }
    for (size_t i = 0; i < g.size(); ++i)
        if ((g[i] != 0) != c[i]) { printf("FAIL %s: [%zu] gpu %d cpu %d\n", what, i, (int)g[i], (int)c[i]); ++fails; return; }
}
static void equal_bits(const char* what, const Tensor& gpu, const Tensor& cpu) {
    ++checks;
    auto g = to_host<float>(gpu);
    if (std::memcmp(g.data(), cpu.data_ptr<float>(), g.size() * 4) != 0) { printf("FAIL %s: bits differ\n", what); ++fails; }
}

int main() {
    setvbuf(stdout, nullptr, _IONBF, 0);
    const int64_t R = 64, C = 1000;
    std::vector<float> v(R * C);
    unsigned s = 12345u;
    for (auto& x : v) { s = s * 1664525u + 1013904223u; x = (float)((int)(s >> 8) % 2001 - 1000) / 250.0f; }
    v[7] = v[3];   // ties
    Tensor c = Tensor::tensor<float>(v).reshape({R, C});
    Tensor g = to_cuda(c);
    if (!g.device().is_cuda()) { printf("FAIL: no CUDA tensor\n"); return 2; }
    const double tol = 2e-3;   // the reference's CPU dim-sum accumulates sequentially in float32
    close_f("sum(dim=1)", g.sum({1}, false, DType::Undefined), c.sum({1}, false, DType::Undefined), 1e-5, tol);
    close_f("sum(dim=0,keepdim)", g.sum({0}, true, DType::Undefined), c.sum({0}, true, DType::Undefined), 1e-5, tol);
    close_f("sum()", g.sum(DType::Undefined), c.sum(DType::Undefined), 1e-5, tol);
    close_f("mean(dim=-1)", g.mean({-1}, false, DType::Undefined), c.mean({-1}, false, DType::Undefined), 1e-5, 1e-5);
    close_f("mean()", g.mean(DType::Undefined), c.mean(DType::Undefined), 1e-5, 1e-6);
    close_f("var(dim=1)", g.var({1}, 1, false), c.var({1}, 1, false), 1e-4, 0);
    close_f("std()", g.std(1), c.std(1), 1e-4, 0);
    equal_bits("max(dim=1)", g.max({1}, false), c.max({1}, false));
    equal_bits("min(dim=0)", g.min({0}, false), c.min({0}, false));
    equal_bits("max()", g.max(), c.max());
    equal_i("argmax(1)", g.argmax(std::optional<int64_t>(1), false), c.argmax(std::optional<int64_t>(1), false));
    equal_i("argmin(0,keepdim)", g.argmin(std::optional<int64_t>(0), true), c.argmin(std::optional<int64_t>(0), true));
    equal_i("argmax()", g.argmax(std::nullopt, false), c.argmax(std::nullopt, false));
    // a strided view (the transpose, built on the same storage) is consumed in place
    Tensor gt(g.impl()->storage(), {C, R}, {1, C}, DType::Float32, 0);
    Tensor ct(c.impl()->storage(), {C, R}, {1, C}, DType::Float32, 0);
    close_f("sum(dim=0) of a transposed view", gt.sum({0}, false, DType::Undefined), ct.sum({0}, false, DType::Undefined), 1e-5, tol);
    equal_i("argmax(1) of a transposed view", gt.argmax(std::optional<int64_t>(1), false), ct.argmax(std::optional<int64_t>(1), false));
    // the other operators of the registration block: prod, norm, all, any
    std::vector<float> w(R * C);
    for (size_t i = 0; i < w.size(); ++i) { s = s * 1664525u + 1013904223u; w[i] = 0.9f + (float)((s >> 8) % 201) / 1000.0f; }
    w[5 * C + 17] = 0.0f;
    Tensor cw = Tensor::tensor<float>(w).reshape({R, C});
    Tensor gw = to_cuda(cw);
    close_f("prod(dim=1)", gw.prod({1}, false, DType::Undefined), cw.prod({1}, false, DType::Undefined), 1e-4, 0);
    close_f("prod()", gw.prod(DType::Undefined), cw.prod(DType::Undefined), 1e-4, 0);
    close_f("norm()", g.norm(2.0), c.norm(2.0), 1e-5, 0);
    close_f("norm(dim=0,p=2,keepdim)", g.norm({0}, 2.0, true), c.norm({0}, 2.0, true), 1e-5, 0);
    close_f("norm(dim=1,p=1)", g.norm({1}, 1.0, false), c.norm({1}, 1.0, false), 1e-5, 0);
    equal_bits("norm(dim=1,p=inf)", g.norm({1}, std::numeric_limits<double>::infinity(), false),
               c.norm({1}, std::numeric_limits<double>::infinity(), false));
    equal_bool("all(dim=1)", gw.all({1}, false), cw.all({1}, false));
    equal_bool("any(dim=0,keepdim)", gw.any({0}, true), cw.any({0}, true));
    equal_bool("all()", gw.all(), cw.all());
    equal_bool("any()", gw.any(), cw.any());
    // topk: not declared by the reference; the schema entry beside the adapter adds Tensor::topk, which
    // must reach the new kernel through the Dispatcher.  Expected values from the CPU checker on the
    // host copy: last dim and a non-last dim, both directions, with ties (v[7] == v[3]) and a
    // tie-heavy row.
    {
        std::vector<float> tv(v);
        for (int64_t j = 0; j < C; ++j) tv[9 * C + j] = (float)(j % 5);       // row 9: 200 copies of each value
        Tensor ct2 = Tensor::tensor<float>(tv).reshape({R, C});
        Tensor gt2 = to_cuda(ct2);
        for (int largest = 0; largest < 2; ++largest) {
            const int64_t k = 17;
            auto [vals, idx] = gt2.topk(k, -1, largest != 0, true);
            std::vector<float> wv(R * k);
            std::vector<int64_t> wi(R * k);
            tpo_topk(tv.data(), R, C, C, 1, k, largest, wv.data(), wi.data());
            ++checks;
            auto hv = to_host<float>(vals);
            auto hi = to_host<int64_t>(idx);
            if (static_cast<std::vector<int64_t>>(vals.shape()) != std::vector<int64_t>{R, k} || idx.dtype() != DType::Int64 ||
                std::memcmp(hv.data(), wv.data(), wv.size() * 4) != 0 || hi != wi) { printf("FAIL topk(dim=-1, largest=%d)\n", largest); ++fails; }
            // along dim 0: rows are the columns of the matrix, read with stride C
            const int64_t k0 = 5;
            auto [vals0, idx0] = gt2.topk(k0, 0, largest != 0, true);
            std::vector<float> wv0(C * k0);
            std::vector<int64_t> wi0(C * k0);
            tpo_topk(tv.data(), C, R, 1, C, k0, largest, wv0.data(), wi0.data());
            ++checks;
            // the result is a [k0, C] view of storage laid out [C, k0]
            auto hv0 = to_host<float>(vals0);
            auto hi0 = to_host<int64_t>(idx0);
            if (static_cast<std::vector<int64_t>>(vals0.shape()) != std::vector<int64_t>{k0, C} || vals0.strides() != std::vector<int64_t>{1, k0} ||
                std::memcmp(hv0.data(), wv0.data(), wv0.size() * 4) != 0 || hi0 != wi0) { printf("FAIL topk(dim=0, largest=%d)\n", largest); ++fails; }
        }
        auto [v1, i1] = Tensor::topk(gt2, 1, 1, true, true);                  // function variant; k = 1 is argmax
        equal_i("topk(k=1) indices == argmax", i1, ct2.argmax(std::optional<int64_t>(1), false));   // [R,1] against [R]: same elements
        try { gt2.topk(C + 1, -1, true, true); printf("FAIL: no error for k > len\n"); ++fails; }
        catch (const std::exception& e) { ++checks; if (!std::strstr(e.what(), "selected index k out of range")) { printf("FAIL: message %s\n", e.what()); ++fails; } }
    }
    // softmax / log_softmax (the reference's CUDA kernels for them are cuDNN calls) and median (CPU only
    // in the reference) through the same Dispatcher
    close_f("softmax(dim=1)", g.softmax(1, DType::Undefined), c.softmax(1, DType::Undefined), 1e-5, 1e-30);
    close_f("softmax(dim=0)", g.softmax(0, DType::Undefined), c.softmax(0, DType::Undefined), 1e-5, 1e-30);
    close_f("log_softmax(dim=-1)", g.log_softmax(-1, DType::Undefined), c.log_softmax(-1, DType::Undefined), 1e-5, 1e-5);
    equal_bits("median()", g.median(), c.median());
    // copy_ of a strided view (what permute().contiguous() runs): the transposed view built above into a
    // fresh contiguous tensor, through the Dispatcher to the tiled copy kernel
    {
        Tensor dstg(std::vector<int64_t>{C, R}, DType::Float32, Device(DeviceType::CUDA, 0));
        dstg.copy_(gt);
        auto h = to_host<float>(dstg);
        ++checks;
        bool ok = true;
        for (int64_t i = 0; i < C && ok; ++i)
            for (int64_t j = 0; j < R; ++j)
                if (std::memcmp(&h[i * R + j], &v[j * C + i], 4) != 0) { ok = false; break; }
        if (!ok) { printf("FAIL copy_ of a transposed view\n"); ++fails; }
    }
    // errors keep the reference's type and message
    try { g.sum({2}, false, DType::Undefined); printf("FAIL: no error for a bad dim\n"); ++fails; }
    catch (const std::exception& e) { ++checks; if (!std::strstr(e.what(), "Dimension out of range")) { printf("FAIL: message %s\n", e.what()); ++fails; } }
    // Through-dispatcher latency: TensorPlay's generated Tensor::sum / Tensor::argmax on a [4096,4096]
    // CUDA tensor, result allocation (the reference's allocator: one cudaMalloc and one cudaFree per
    // call) and scratch included, against the device time of the kernel alone.
    {
        const int64_t N = 4096;
        Tensor big(std::vector<int64_t>{N, N}, DType::Float32, Device(DeviceType::CUDA, 0));
        cudaMemset(big.data_ptr(), 0, (size_t)N * N * 4);
        cudaEvent_t e0, e1;
        cudaEventCreate(&e0); cudaEventCreate(&e1);
        for (int which = 0; which < 2; ++which) {
            for (int i = 0; i < 5; ++i) { Tensor r = which ? big.argmax(std::optional<int64_t>(1), false) : big.sum({1}, false, DType::Undefined); }
            cudaDeviceSynchronize();
            const int iters = 200;
            timespec t0, t1;
            clock_gettime(CLOCK_MONOTONIC, &t0);
            for (int i = 0; i < iters; ++i) { Tensor r = which ? big.argmax(std::optional<int64_t>(1), false) : big.sum({1}, false, DType::Undefined); }
            cudaDeviceSynchronize();
            clock_gettime(CLOCK_MONOTONIC, &t1);
            const double wall_us = ((t1.tv_sec - t0.tv_sec) * 1e9 + (t1.tv_nsec - t0.tv_nsec)) / 1e3 / iters;
            printf("dispatcher_latency %s [4096,4096] dim=1: %.1f us per call through Tensor::%s (allocation included)\n",
                   which ? "argmax" : "sum", wall_us, which ? "argmax" : "sum");
        }
        cudaEventDestroy(e0); cudaEventDestroy(e1);
    }
    printf("adapter_check: %d checks, %d failures\n", checks, fails);
    fflush(stdout);
    return fails ? 1 : 0;
}
