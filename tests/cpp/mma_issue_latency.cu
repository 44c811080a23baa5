// Microbenchmark: what the thread that issues tcgen05.mma pays for the instructions between two groups of MMAs.
//
// One thread per CTA issues 512 groups of MMAs (M = 128, K = 16, operands in shared memory, fp32 accumulator in
// TMEM) and the kernel reports SM cycles per group for several kinds of instruction placed between the groups.
// The numbers explain the stage sizes of the kernels in tiledcuda_b200/csrc: the tensor pipe runs barely one or
// two MMAs behind the issuing thread, so a barrier wait between short MMAs leaves it idle.
// Every wait is bounded (sm100.cuh); the operands are whatever shared memory holds, the results are discarded.
//
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -o mma_issue_latency mma_issue_latency.cu
#include <cstdio>
#include <cuda_runtime.h>

#include "../../tiledcuda_b200/csrc/sm100.cuh"

using namespace tcb;

enum Between { kNothing, kCommit, kFence, kSharedLoad, kTestWait, kTryWait, kRing };

template <int NN, int STAGES, int BETWEEN, int MMAS>
__global__ void __launch_bounds__(64, 1) issue_loop(long long* out, int groups) {
    extern __shared__ uint8_t raw[];
    uint8_t* smem = align_smem_1024(raw);
    uint64_t* bar_full = reinterpret_cast<uint64_t*>(smem + 192 * 1024);
    uint64_t* bar_empty = bar_full + STAGES;
    uint64_t* bar_done = bar_empty + STAGES;
    uint32_t* slot = reinterpret_cast<uint32_t*>(bar_done + 1);
    volatile uint32_t* abort_word = slot + 1;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&bar_full[s], 1);
            mbar_init(&bar_empty[s], 1);
        }
        mbar_init(bar_done, 1);
        *abort_word = 0;
        fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc(slot, 512);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *slot;
    if (warp == 0 && lane == 0 && BETWEEN == kRing) {
        // the producer of a ring: waits for a free stage and reports it full (no data is moved)
        int stage = 0;
        uint32_t phase = 0;
        for (int g = 0; g < groups; ++g) {
            if (!mbar_wait(&bar_empty[stage], phase ^ 1u, abort_word, 1)) break;
            mbar_arrive(&bar_full[stage]);
            if (++stage == STAGES) {
                stage = 0;
                phase ^= 1u;
            }
        }
    } else if (warp == 1) {
        const long long t0 = clock64();
        if (lane == 0) {
            const uint32_t idesc = make_idesc_f16_f32(128, NN, false, false);
            int stage = 0;
            uint32_t phase = 0;
            for (int g = 0; g < groups; ++g) {
                // a wait with parity 1 on a barrier that was never used returns at once: "completed phase"
                if (BETWEEN == kRing && !mbar_wait(&bar_full[stage], phase, abort_word, 2)) break;
                if (BETWEEN == kTryWait && !mbar_wait(&bar_full[stage], 1u, abort_word, 2)) break;
                if (BETWEEN == kTestWait && !mbar_test(&bar_full[stage], 1u)) break;
                if (BETWEEN == kSharedLoad && *abort_word != 0) break;
                if (BETWEEN == kFence || BETWEEN == kRing) tc_fence_after_sync();
                const uint64_t a_desc = make_smem_desc_sw128(smem_u32(smem + stage * 16384), 16, 1024);
                const uint64_t b_desc = make_smem_desc_sw128(smem_u32(smem + 98304 + stage * 8192), 16, 1024);
#pragma unroll
                for (int k = 0; k < MMAS; ++k)
                    umma_f16_ss(tmem, a_desc + static_cast<uint64_t>((k & 3) * 2), b_desc + static_cast<uint64_t>((k & 3) * 2),
                                idesc, (g | k) != 0);
                if (BETWEEN == kCommit || BETWEEN == kRing) umma_commit(&bar_empty[stage]);
                if (++stage == STAGES) {
                    stage = 0;
                    phase ^= 1u;
                }
            }
            umma_commit(bar_done);
        }
        __syncwarp();
        mbar_wait_warp(bar_done, 0, abort_word, 3);
        const long long t1 = clock64();
        if (lane == 0 && blockIdx.x == 0) {
            out[0] = t1 - t0;
            out[1] = *abort_word;
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem, 512);
    }
}

template <int NN, int STAGES, int BETWEEN, int MMAS>
static int run(const char* what) {
    long long* d = nullptr;
    long long h[2] = {0, 0};
    if (cudaMalloc(&d, 16) != cudaSuccess) return 1;
    auto kernel = issue_loop<NN, STAGES, BETWEEN, MMAS>;
    cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    const int groups = 512;
    for (int rep = 0; rep < 2; ++rep) {
        kernel<<<8, 64, 200 * 1024>>>(d, groups);
        if (cudaDeviceSynchronize() != cudaSuccess) break;
    }
    const cudaError_t err = cudaGetLastError();
    cudaMemcpy(h, d, 16, cudaMemcpyDeviceToHost);
    cudaFree(d);
    printf("N=%d mmas_per_group=%d between=%s cycles_per_group=%.0f status=%lld %s\n", NN, MMAS, what, h[0] / double(groups), h[1],
           cudaGetErrorString(err));
    return err == cudaSuccess && h[1] == 0 ? 0 : 1;
}

int main() {
    int bad = 0;
    bad += run<64, 4, kNothing, 4>("nothing");
    bad += run<64, 4, kCommit, 4>("commit");
    bad += run<64, 4, kFence, 4>("fence");
    bad += run<64, 4, kSharedLoad, 4>("shared_load");
    bad += run<64, 4, kTestWait, 4>("test_wait");
    bad += run<64, 4, kTryWait, 4>("try_wait");
    bad += run<64, 4, kRing, 4>("ring");
    bad += run<64, 4, kTryWait, 8>("try_wait");
    bad += run<64, 4, kTryWait, 16>("try_wait");
    bad += run<128, 4, kNothing, 4>("nothing");
    bad += run<128, 4, kTryWait, 4>("try_wait");
    bad += run<128, 4, kRing, 4>("ring");
    bad += run<256, 4, kNothing, 4>("nothing");
    bad += run<256, 4, kTryWait, 4>("try_wait");
    bad += run<256, 4, kRing, 4>("ring");
    return bad;
}
