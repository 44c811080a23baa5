// BASELINE INFRASTRUCTURE ONLY (never linked into the product): runs the reference's own library attention kernel
// (src/kernels/flash_attn.cu, included from the reference tree where it lies) at the largest of the three shapes its
// launcher supports, m = 64, n = 256, k = p = 128 (flash_attn.cu:438-455), through its own run_flash_attention with
// its own CTA tile 64 x 64 x 128 x 128. Layouts as the reference takes them: Q [m,k] rows, K as [n,k] rows, V as V^T
// [p,n] rows, O [m,p] rows, fp16. The result is compared on the host with softmax(Q K^T) V in fp32 (the bound is the
// reference test's own 8e-2, tests/python/test_flash_attn.py:114), then the call is timed; the reference's launcher
// synchronises the device inside every call (flash_attn.cu:421), so the time is per synchronous call.
//
// Prints one line:  REF_FA m=64 n=256 k=128 p=128 us=<per call> gflops=<..> check=<ok|FAILED> max_abs_err=<..>
#include "flash_attn.cu"

#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <vector>

int main() {
    constexpr int m = 64, n = 256, k = 128, p = 128;
    std::vector<__half> hq(m * k), hk(n * k), hvt(p * n), ho(m * p);
    srand(1234);
    auto rnd = [] { return 2.f * rand() / RAND_MAX - 1.f; };
    for (auto& x : hq) x = __float2half(rnd());
    for (auto& x : hk) x = __float2half(rnd());
    for (auto& x : hvt) x = __float2half(rnd());
    __half *dq, *dk, *dv, *dout;
    if (cudaMalloc(&dq, hq.size() * 2) != cudaSuccess || cudaMalloc(&dk, hk.size() * 2) != cudaSuccess ||
        cudaMalloc(&dv, hvt.size() * 2) != cudaSuccess || cudaMalloc(&dout, ho.size() * 2) != cudaSuccess) {
        printf("REF_FA unavailable: cudaMalloc failed\n");
        return 1;
    }
    cudaMemcpy(dq, hq.data(), hq.size() * 2, cudaMemcpyHostToDevice);
    cudaMemcpy(dk, hk.data(), hk.size() * 2, cudaMemcpyHostToDevice);
    cudaMemcpy(dv, hvt.data(), hvt.size() * 2, cudaMemcpyHostToDevice);
    cudaMemset(dout, 0, ho.size() * 2);

    using Whole = tiledcuda::kernels::FlashAttentionShape<m, n, k, p>;
    using Cta = TileShape<64, 64, 128, 128>;
    auto call = [&] { tiledcuda::kernels::run_flash_attention<__half, float, __half, Whole, Cta, 1>(dq, dk, dv, dout); };
    call();
    cudaError_t err = cudaDeviceSynchronize();
    if (err != cudaSuccess) {
        printf("REF_FA unavailable: %s\n", cudaGetErrorString(err));
        return 1;
    }
    cudaMemcpy(ho.data(), dout, ho.size() * 2, cudaMemcpyDeviceToHost);
    double max_err = 0.;
    std::vector<float> s(n);
    for (int i = 0; i < m; ++i) {
        float mx = -1e30f;
        for (int j = 0; j < n; ++j) {
            float acc = 0.f;
            for (int t = 0; t < k; ++t) acc += __half2float(hq[i * k + t]) * __half2float(hk[j * k + t]);
            s[j] = acc;
            mx = fmaxf(mx, acc);
        }
        float sum = 0.f;
        for (int j = 0; j < n; ++j) sum += (s[j] = expf(s[j] - mx));
        for (int c = 0; c < p; ++c) {
            float acc = 0.f;
            for (int j = 0; j < n; ++j) acc += s[j] * __half2float(hvt[c * n + j]);
            const double e = std::fabs(acc / sum - __half2float(ho[i * p + c]));
            if (e > max_err) max_err = e;
        }
    }
    for (int i = 0; i < 10; ++i) call();
    const int iters = 50;
    const auto t0 = std::chrono::steady_clock::now();
    for (int i = 0; i < iters; ++i) call();
    const double us = std::chrono::duration<double, std::micro>(std::chrono::steady_clock::now() - t0).count() / iters;
    printf("REF_FA m=%d n=%d k=%d p=%d us=%.2f gflops=%.1f check=%s max_abs_err=%.3e\n", m, n, k, p, us, 4.0 * m * n * k / us / 1e3,
           max_err <= 8e-2 ? "ok" : "FAILED", max_err);
    return 0;
}
