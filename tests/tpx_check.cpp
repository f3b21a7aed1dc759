// TEST INFRASTRUCTURE.  TensorPlay's autograd (TPX) on CUDA tensors, with the reduction kernels of this
// repository registered through tensorplay_b200/csrc/adapter/: the backward nodes that
// config/derivatives.yaml:82-86,182-186 generates for sum / mean / var / std (their formulas call
// mean() and numel()) and AccumulateGrad's un-broadcasting (tpx/include/AccumulateGrad.h:55-60 calls
// ops::sum(grad, dims, false)) must reach the new kernels unchanged and give the right gradients.
// Everything but the reductions is the reference's own code: its engine, its generated nodes and its
// CUDA kernels for expand / add / mul / div / fill.  Built by oracle/build_tpx_check.sh against a
// TensorPlay checkout; run by tests/test_gpu_adapter.py.
#include "TPXTensor.h"
#include "Autograd.h"
#include "tensorplay/ops/TPXOpsGenerated.h"

#include <cuda_runtime.h>

#include <cmath>
#include <cstdio>
#include <vector>

using namespace tensorplay;
extern "C" long long tpb200_adapter_calls(void);

static int fails = 0, checks = 0;

static tpx::Tensor cuda_leaf(const std::vector<float>& v, const std::vector<int64_t>& shape, bool requires_grad) {
    tensorplay::Tensor g(shape, DType::Float32, Device(DeviceType::CUDA, 0));
    cudaMemcpy(g.data_ptr(), v.data(), v.size() * sizeof(float), cudaMemcpyHostToDevice);
    tpx::Tensor t(g);
    if (requires_grad) t.set_requires_grad(true);
    return t;
}
static std::vector<float> host(const tpx::Tensor& t) {
    tensorplay::Tensor c = t.core().is_contiguous() ? t.core() : t.core().clone();
    std::vector<float> h(c.numel());
    cudaDeviceSynchronize();
    cudaMemcpy(h.data(), c.data_ptr(), h.size() * sizeof(float), cudaMemcpyDeviceToHost);
    return h;
}
static void expect(const char* what, const std::vector<float>& got, const std::vector<double>& want, double rel) {
    ++checks;
    if (got.size() != want.size()) { printf("FAIL %s: %zu values, expected %zu\n", what, got.size(), want.size()); ++fails; return; }
    for (size_t i = 0; i < got.size(); ++i)
        if (!(std::fabs(got[i] - want[i]) <= rel * std::fabs(want[i]) + 1e-7)) {
            printf("FAIL %s: [%zu] %.9g expected %.9g\n", what, i, got[i], want[i]); ++fails; return;
        }
}
static void expect_calls(const char* what, long long before, long long at_least) {
    ++checks;
    const long long n = tpb200_adapter_calls() - before;
    if (n < at_least) { printf("FAIL %s: %lld calls reached the new kernels, expected at least %lld\n", what, n, at_least); ++fails; }
}

int main() {
    setvbuf(stdout, nullptr, _IONBF, 0);
    const int64_t R = 48, C = 500, N = R * C;
    std::vector<float> v(N);
    unsigned s = 777u;
    for (auto& x : v) { s = s * 1664525u + 1013904223u; x = (float)((int)(s >> 9) % 4001 - 2000) / 500.0f; }
    double mean = 0;
    for (float x : v) mean += x;
    mean /= N;

    {   // sum: SumBackward = grad.expand(self.shape())
        tpx::Tensor x = cuda_leaf(v, {R, C}, true);
        long long c0 = tpb200_adapter_calls();
        tpx::Tensor y = x.sum();
        expect_calls("forward sum()", c0, 1);
        tpx::backward(y);
        expect("d sum / dx", host(x.grad()), std::vector<double>(N, 1.0), 1e-6);
    }
    {   // mean: MeanBackward = grad.expand(self.shape()) / self.numel()
        tpx::Tensor x = cuda_leaf(v, {R, C}, true);
        long long c0 = tpb200_adapter_calls();
        tpx::Tensor y = x.mean();
        expect_calls("forward mean()", c0, 1);
        tpx::backward(y);
        expect("d mean / dx", host(x.grad()), std::vector<double>(N, 1.0 / N), 1e-5);
    }
    {   // var: VarBackward = grad * 2 * (self - self.mean()) / (self.numel() - correction): mean() runs in backward
        tpx::Tensor x = cuda_leaf(v, {R, C}, true);
        tpx::Tensor y = x.var(1);
        long long c0 = tpb200_adapter_calls();
        tpx::backward(y);
        expect_calls("backward of var(): self.mean()", c0, 1);
        std::vector<double> want(N);
        for (int64_t i = 0; i < N; ++i) want[i] = 2.0 * (v[i] - mean) / (double)(N - 1);
        expect("d var / dx", host(x.grad()), want, 1e-4);
    }
    {   // AccumulateGrad: a [1, C] parameter broadcast against [R, C]; its gradient arrives as [R, C] and is
        // summed over dim 0 by ops::sum(grad, {0}, false) -- a dim reduction on CUDA, i.e. the new kernel
        std::vector<float> pv(C, 0.5f);
        tpx::Tensor p = cuda_leaf(pv, {1, C}, true);
        tpx::Tensor b = cuda_leaf(v, {R, C}, false);
        tpx::Tensor z = (p + b).sum();
        long long c0 = tpb200_adapter_calls();
        tpx::backward(z);
        expect_calls("AccumulateGrad un-broadcast sum", c0, 1);
        expect("d sum(p + b) / dp", host(p.grad()), std::vector<double>(C, (double)R), 1e-6);
    }
    // The dim variants get graph nodes from the additive formulas of
    // tensorplay_b200/csrc/adapter/derivatives_add.yaml (the reference has formulas for the whole-tensor
    // overloads only): forward and backward both run reductions over a dim on CUDA.
    {
        tpx::Tensor x = cuda_leaf(v, {R, C}, true);
        long long c0 = tpb200_adapter_calls();
        tpx::Tensor z = x.sum({1}, false).sum();
        expect_calls("forward sum(dim=1).sum()", c0, 2);
        tpx::backward(z);
        expect("d sum(dim=1).sum() / dx", host(x.grad()), std::vector<double>(N, 1.0), 1e-6);
    }
    {
        tpx::Tensor x = cuda_leaf(v, {R, C}, true);
        tpx::Tensor z = x.mean({0}, true).sum();
        tpx::backward(z);
        expect("d mean(dim=0, keepdim).sum() / dx", host(x.grad()), std::vector<double>(N, 1.0 / R), 1e-5);
    }
    {
        tpx::Tensor x = cuda_leaf(v, {R, C}, true);
        tpx::Tensor z = x.var({1}, 1, false).sum();
        long long c0 = tpb200_adapter_calls();
        tpx::backward(z);
        expect_calls("backward of var(dim=1): self.mean(dim, true)", c0, 1);
        std::vector<double> want(N);
        for (int64_t r = 0; r < R; ++r) {
            double m = 0;
            for (int64_t j = 0; j < C; ++j) m += v[r * C + j];
            m /= C;
            for (int64_t j = 0; j < C; ++j) want[r * C + j] = 2.0 * (v[r * C + j] - m) / (double)(C - 1);
        }
        expect("d var(dim=1).sum() / dx", host(x.grad()), want, 1e-4);
    }
    {
        tpx::Tensor x = cuda_leaf(v, {R, C}, true);
        tpx::Tensor z = x.std({1}, 1, false).sum();
        tpx::backward(z);
        std::vector<double> want(N);
        for (int64_t r = 0; r < R; ++r) {
            double m = 0, q = 0;
            for (int64_t j = 0; j < C; ++j) m += v[r * C + j];
            m /= C;
            for (int64_t j = 0; j < C; ++j) q += (v[r * C + j] - m) * (v[r * C + j] - m);
            const double sd = std::sqrt(q / (C - 1));
            for (int64_t j = 0; j < C; ++j) want[r * C + j] = (v[r * C + j] - m) / (sd * (C - 1));
        }
        expect("d std(dim=1).sum() / dx", host(x.grad()), want, 1e-4);
    }
    printf("tpx_check: %d checks, %d failures\n", checks, fails);
    return fails ? 1 : 0;
}
