// GEMM with host-resident operands: C_host = A_host * B_host, the copies pipelined against the kernel.
//
// A call with host buffers is dominated by PCIe: at 8192^3 the operands are 256 MiB in and the result is
// 256 MiB out, against under a millisecond of tensor-core time. The two directions of the link are
// independent, so the work is cut into blocks C(i, j) = A_i * B_j (row slabs of A, row slabs of the [N, K]
// B): slabs go up in the order A_0, B_0, B_1, A_1, B_2, A_2, ..., a block is multiplied on the compute stream as
// soon as both of its slabs have landed, and its result starts down the other direction immediately. The
// first result leaves after two slabs instead of after both operands, and uploads, products and downloads
// overlap from then on. Streams and events are created once per device and reused; the device staging
// memory is the caller's (no allocation here). Host buffers should be pinned, otherwise the copies are
// staged by the driver and do not overlap.
#include <mutex>
#include <stdio.h>
#include <stdlib.h>

#include "host.h"

namespace tcb {

constexpr int kHostMaxSlabs = 8;

struct HostPipe {
    bool ready = false;
    cudaStream_t s_in = nullptr, s_out = nullptr;
    cudaEvent_t start = nullptr, done = nullptr;
    cudaEvent_t a_in[kHostMaxSlabs], b_in[kHostMaxSlabs];
    cudaEvent_t blk[kHostMaxSlabs * kHostMaxSlabs];
};
static HostPipe g_pipe[64];
static std::mutex g_pipe_mu;

static int get_pipe(HostPipe** out) {
    int dev = -1;
    TCB_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(TC_ERR_UNSUPPORTED, "device ordinal %d out of range", dev);
    std::lock_guard<std::mutex> lock(g_pipe_mu);
    HostPipe& p = g_pipe[dev];
    if (!p.ready) {
        TCB_CUDA(cudaStreamCreateWithFlags(&p.s_in, cudaStreamNonBlocking));
        TCB_CUDA(cudaStreamCreateWithFlags(&p.s_out, cudaStreamNonBlocking));
        TCB_CUDA(cudaEventCreateWithFlags(&p.start, cudaEventDisableTiming));
        TCB_CUDA(cudaEventCreateWithFlags(&p.done, cudaEventDisableTiming));
        for (int i = 0; i < kHostMaxSlabs; ++i) {
            TCB_CUDA(cudaEventCreateWithFlags(&p.a_in[i], cudaEventDisableTiming));
            TCB_CUDA(cudaEventCreateWithFlags(&p.b_in[i], cudaEventDisableTiming));
        }
        for (int i = 0; i < kHostMaxSlabs * kHostMaxSlabs; ++i) TCB_CUDA(cudaEventCreateWithFlags(&p.blk[i], cudaEventDisableTiming));
        p.ready = true;
    }
    *out = &p;
    return TC_OK;
}

static int64_t slab_rows(int64_t total, int slabs) {
    const int64_t per = (total + slabs - 1) / slabs;
    return (per + 255) / 256 * 256;  // whole 256-row tiles, so every block takes the same kernel path
}

}  // namespace tcb

extern "C" int64_t tc_gemm_host_workspace_bytes(int64_t M, int64_t N, int64_t K) {
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    return M * K * 2 + N * K * 2 + M * N * 4;
}

extern "C" int tc_gemm_f16_f32_host(const void* hA, const void* hB, void* hC, int64_t M, int64_t N, int64_t K,
                                    void* d_workspace, int64_t workspace_bytes, tc_stream_t stream) {
    using namespace tcb;
    TCB_REQUIRE(hA && hB && hC && d_workspace, "gemm_host: null pointer argument");
    TCB_REQUIRE(M > 0 && N > 0 && K > 0 && K % 8 == 0, "gemm_host: M, N, K must be positive and K a multiple of 8");
    TCB_REQUIRE(workspace_bytes >= tc_gemm_host_workspace_bytes(M, N, K), "gemm_host: workspace holds %lld bytes, %lld needed",
                (long long)workspace_bytes, (long long)tc_gemm_host_workspace_bytes(M, N, K));
    TCB_REQUIRE((reinterpret_cast<uintptr_t>(d_workspace) & 255u) == 0, "gemm_host: workspace must be 256-byte aligned");
    HostPipe* p = nullptr;
    if (int rc = get_pipe(&p)) return rc;
    auto* st = static_cast<cudaStream_t>(stream);

    auto* dA = static_cast<uint8_t*>(d_workspace);
    auto* dB = dA + M * K * 2;
    auto* dC = dB + N * K * 2;
    TCB_REQUIRE((reinterpret_cast<uintptr_t>(dB) & 15u) == 0 && (reinterpret_cast<uintptr_t>(dC) & 15u) == 0,
                "gemm_host: M*K and N*K must keep the staging areas 16-byte aligned");
    const int sa = static_cast<int>(M >= 2048 ? (M >= 8192 ? 4 : 2) : 1);
    const int sb = static_cast<int>(N >= 2048 ? (N >= 8192 ? 4 : 2) : 1);
    const int64_t ra = slab_rows(M, sa), rb = slab_rows(N, sb);

    // uploads follow everything already queued on the caller's stream
    TCB_CUDA(cudaEventRecord(p->start, st));
    TCB_CUDA(cudaStreamWaitEvent(p->s_in, p->start, 0));
    TCB_CUDA(cudaStreamWaitEvent(p->s_out, p->start, 0));

    auto upload_a = [&](int i) -> int {
        const int64_t r0 = i * ra, rows = (r0 + ra <= M ? ra : M - r0);
        if (rows <= 0) return TC_OK;
        TCB_CUDA(cudaMemcpyAsync(dA + r0 * K * 2, static_cast<const uint8_t*>(hA) + r0 * K * 2, rows * K * 2, cudaMemcpyHostToDevice, p->s_in));
        TCB_CUDA(cudaEventRecord(p->a_in[i], p->s_in));
        return TC_OK;
    };
    auto upload_b = [&](int j) -> int {
        const int64_t r0 = j * rb, rows = (r0 + rb <= N ? rb : N - r0);
        if (rows <= 0) return TC_OK;
        TCB_CUDA(cudaMemcpyAsync(dB + r0 * K * 2, static_cast<const uint8_t*>(hB) + r0 * K * 2, rows * K * 2, cudaMemcpyHostToDevice, p->s_in));
        TCB_CUDA(cudaEventRecord(p->b_in[j], p->s_in));
        return TC_OK;
    };
    auto block = [&](int i, int j) -> int {
        const int64_t m0 = i * ra, n0 = j * rb;
        const int64_t rows = (m0 + ra <= M ? ra : M - m0), cols = (n0 + rb <= N ? rb : N - n0);
        if (rows <= 0 || cols <= 0) return TC_OK;
        TCB_CUDA(cudaStreamWaitEvent(st, p->a_in[i], 0));
        TCB_CUDA(cudaStreamWaitEvent(st, p->b_in[j], 0));
        float* c_blk = reinterpret_cast<float*>(dC) + m0 * N + n0;
        if (int rc = tc_gemm_f16_f32(dA + m0 * K * 2, dB + n0 * K * 2, c_blk, rows, cols, K, K, K, N, st)) return rc;
        cudaEvent_t ev = p->blk[i * kHostMaxSlabs + j];
        TCB_CUDA(cudaEventRecord(ev, st));
        TCB_CUDA(cudaStreamWaitEvent(p->s_out, ev, 0));
        TCB_CUDA(cudaMemcpy2DAsync(static_cast<float*>(hC) + m0 * N + n0, N * sizeof(float), c_blk, N * sizeof(float),
                                   cols * sizeof(float), rows, cudaMemcpyDeviceToHost, p->s_out));
        return TC_OK;
    };

    // Upload order A_0, B_0, B_1, A_1, B_2, A_2, ...: after each new slab, every block it completes is issued.
    const int steps = sa > sb ? sa : sb;
    for (int s = 0; s < steps; ++s) {
        if (s < sa) {
            if (int rc = upload_a(s)) return rc;
        }
        if (s < sb) {
            if (int rc = upload_b(s)) return rc;
        }
        for (int j = 0; j <= s && j < sb; ++j) {   // new row slab s against all B slabs present
            if (s < sa) {
                if (int rc = block(s, j)) return rc;
            }
        }
        for (int i = 0; i < s && i < sa; ++i) {    // new B slab s against the earlier row slabs
            if (s < sb) {
                if (int rc = block(i, s)) return rc;
            }
        }
    }
    // the caller's stream is done when the last download is
    TCB_CUDA(cudaEventRecord(p->done, p->s_out));
    TCB_CUDA(cudaStreamWaitEvent(st, p->done, 0));
    return TC_OK;
}
