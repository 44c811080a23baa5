// BASELINE INFRASTRUCTURE ONLY (never linked into the product): instantiates the reference's own GEMM kernel
// `gemm` and its `KeGemmTraits` (examples/cpp/01_gemm/02_gemm_all_mem/gemm.hpp, included from the reference tree
// where it lies) at a square problem size given at compile time with -DREF_N=<n>, because the reference fixes the
// size as template constants (its main.cu:5 has 4096^3 only). Same CTA tile (64 x 256 x 32), warp layout and
// register K step as the reference's main.cu:5-8; same timing pattern (10 warm-up + 20 timed launches,
// main.cu:91-103). A sample of output entries is checked against an fp32 dot product on the host.
//
// Prints one line:  REF_GEMM n=<n> ms=<per launch> tflops=<..> check=<ok|FAILED> max_rel_err=<..>
#include "gemm.hpp"

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <vector>

#ifndef REF_N
#define REF_N 8192
#endif

int main() {
    constexpr int kN = REF_N;
    using WholeShape = GemmShape<kN, kN, kN>;
    using CtaTileShape = GemmShape<64, 256, 32>;
    using WarpLayout = tl::RowMajor<2, 2>;
    constexpr int kRK = 32;
    constexpr int kTM = 64, kTN = 256, kTK = 32;
    using Config = KeGemmTraits<__half, float, WholeShape, CtaTileShape, kRK, WarpLayout>;
    auto kernel = &gemm<__half, float, kN, kN, kN, kTM, kTN, kTK, typename Config::GIteratorA, typename Config::SIteratorA,
                        typename Config::SharedA, typename Config::RegA, typename Config::G2SLoaderA, typename Config::S2RLoaderA,
                        typename Config::GIteratorB, typename Config::SIteratorB, typename Config::SharedB, typename Config::RegB,
                        typename Config::G2SLoaderB, typename Config::S2RLoaderB, typename Config::GlobalC, typename Config::SharedC,
                        typename Config::RegC, typename Config::R2SStorerC, typename Config::S2GStorerC>;

    const size_t elems = static_cast<size_t>(kN) * kN;
    std::vector<__half> h_a(elems), h_b(elems);
    srand(1234);
    for (size_t i = 0; i < elems; ++i) h_a[i] = __float2half(2.f * rand() / RAND_MAX - 1.f);   // uniform [-1, 1)
    for (size_t i = 0; i < elems; ++i) h_b[i] = __float2half(2.f * rand() / RAND_MAX - 1.f);
    __half *d_a = nullptr, *d_b = nullptr;
    float* d_c = nullptr;
    if (cudaMalloc(&d_a, elems * 2) != cudaSuccess || cudaMalloc(&d_b, elems * 2) != cudaSuccess ||
        cudaMalloc(&d_c, elems * 4) != cudaSuccess) {
        printf("REF_GEMM n=%d unavailable: cudaMalloc failed\n", kN);
        return 1;
    }
    cudaMemcpy(d_a, h_a.data(), elems * 2, cudaMemcpyHostToDevice);
    cudaMemcpy(d_b, h_b.data(), elems * 2, cudaMemcpyHostToDevice);
    cudaMemset(d_c, 0, elems * 4);

    constexpr int smem_inputs = kTK * (kTN + kTM) * 2;
    constexpr int smem_acc = kTM * kTN * 4;
    constexpr int smem = smem_inputs > smem_acc ? smem_inputs : smem_acc;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    const dim3 grid(kN / kTM, kN / kTN, 1), block(Config::kThreads, 1, 1);

    kernel<<<grid, block, smem>>>(d_a, d_b, d_c);
    cudaError_t err = cudaDeviceSynchronize();
    if (err != cudaSuccess) {
        printf("REF_GEMM n=%d unavailable: %s\n", kN, cudaGetErrorString(err));
        return 1;
    }
    // spot check: 64 entries spread over the matrix against an fp32 dot product of the fp16 inputs
    double max_rel = 0.;
    for (int s = 0; s < 64; ++s) {
        const int i = static_cast<int>((static_cast<long long>(s) * 2654435761ll) % kN);
        const int j = static_cast<int>((static_cast<long long>(s + 17) * 40503ll * 65537ll) % kN);
        float got = 0.f;
        cudaMemcpy(&got, d_c + static_cast<size_t>(i) * kN + j, 4, cudaMemcpyDeviceToHost);
        double want = 0.;
        for (int k = 0; k < kN; ++k)
            want += static_cast<double>(__half2float(h_a[static_cast<size_t>(i) * kN + k])) * __half2float(h_b[static_cast<size_t>(j) * kN + k]);
        const double rel = std::fabs(got - want) / (std::fabs(want) + 1.0);
        if (rel > max_rel) max_rel = rel;
    }

    for (int i = 0; i < 10; ++i) kernel<<<grid, block, smem>>>(d_a, d_b, d_c);
    cudaDeviceSynchronize();
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    const int iters = 20;
    cudaEventRecord(e0);
    for (int i = 0; i < iters; ++i) kernel<<<grid, block, smem>>>(d_a, d_b, d_c);
    cudaEventRecord(e1);
    cudaEventSynchronize(e1);
    float ms = 0.f;
    cudaEventElapsedTime(&ms, e0, e1);
    ms /= iters;
    printf("REF_GEMM n=%d ms=%.4f tflops=%.1f check=%s max_rel_err=%.2e\n", kN, ms, 2.0 * kN * kN * kN / ms / 1e9,
           max_rel < 1e-3 ? "ok" : "FAILED", max_rel);
    cudaFree(d_a);
    cudaFree(d_b);
    cudaFree(d_c);
    return 0;
}
