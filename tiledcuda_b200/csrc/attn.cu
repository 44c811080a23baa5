// FlashAttention-2 forward for sequences longer than one tile: two 128-row Q tiles per CTA, ping-pong.
//
//   warp 0       TMA producer: both Q tiles once, then K_0, V_0, K_1, V_1, ... through one 4-stage ring;
//   warp 1       tcgen05.mma issuer. For each KV block j and each tile t: O_t += P_t(j) V_j (A operand read
//                from TMEM), then S_t = Q_t K_{j+1}^T. While tile 0's scores are being exponentiated the
//                tensor pipe works on tile 1 and vice versa;
//   warps 2..5   softmax warpgroup of tile 0, warps 6..9 of tile 1: one thread per query row. tcgen05.ld
//                the fp32 scores, online softmax with fp32 running maximum and sum (exp2, scale folded
//                in), round to fp16 and tcgen05.st P over the columns the scores came from: P never
//                leaves TMEM. O_t stays in TMEM, is rescaled only when the row maximum grew by more
//                than 2^8, and is normalised once at the end.
// TMEM: S_0 | S_1 | O_0 | O_1, 128 columns each. tcgen05.mma instructions of one CTA execute in issue
// order, so S_t(j+1) may overwrite P_t(j) right after P_t(j) V_j was issued.
//
// Stands in for flash_attention (src/kernels/flash_attn.cu:134-312), which holds one 64-row tile per
// CTA, re-loads Q for every KV block, keeps its statistics in fp16 and divides O by the running sum in
// every block.
#include <math.h>

#include "host.h"
#include "sm100.cuh"

namespace tcb {

constexpr int kFaBM = 128;
constexpr int kFaBN = 128;
constexpr int kFaStages = 4;
constexpr int kFaThreads = 320;
constexpr int kFaTile = 128 * 128 * 2;
constexpr int kFaChunk = 128 * 64 * 2;
constexpr int kFaSmem = kFaTile * (2 + kFaStages) + 256 + 1024;
constexpr float kFaRescaleThreshold = 8.0f;

struct AttnParams {
    int seq_q;
    int seq_kv;
    int dk;
    int dv;
    float scale_log2;
    __half* out;
    float* lse;
    uint32_t* status;
};

template <bool kVTrans>
__global__ void __launch_bounds__(kFaThreads, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                const __grid_constant__ CUtensorMap tmap_v, const AttnParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = align_smem_1024(smem_raw);
    uint8_t* s_q = smem;                   // two Q tiles
    uint8_t* s_kv = smem + 2 * kFaTile;    // ring of K / V tiles
    uint64_t* bars = reinterpret_cast<uint64_t*>(s_kv + kFaStages * kFaTile);
    uint64_t* bar_q_full = bars;                        // 2
    uint64_t* bar_kv_full = bars + 2;                   // kFaStages
    uint64_t* bar_kv_empty = bar_kv_full + kFaStages;   // kFaStages
    uint64_t* bar_s_full = bar_kv_empty + kFaStages;    // 2
    uint64_t* bar_p_full = bar_s_full + 2;              // 2
    uint64_t* bar_o_full = bar_p_full + 2;              // 2
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_o_full + 2);
    volatile uint32_t* abort_word = tmem_slot + 1;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int q0 = blockIdx.x * (2 * kFaBM);
    const int bh = blockIdx.y;
    const int n_blocks = (p.seq_kv + kFaBN - 1) / kFaBN;
    const int k_chunks = (p.dk + 63) / 64;
    const int v_chunks = (p.dv + 63) / 64;
    const int k_steps = p.dk / 16;
    const bool two_tiles = q0 + kFaBM < p.seq_q;  // the second tile may lie wholly outside the sequence

    if (threadIdx.x == 0) {
        for (int t = 0; t < 2; ++t) {
            mbar_init(&bar_q_full[t], 1);
            mbar_init(&bar_s_full[t], 1);
            mbar_init(&bar_p_full[t], 4);
            mbar_init(&bar_o_full[t], 1);
        }
        for (int s = 0; s < kFaStages; ++s) {
            mbar_init(&bar_kv_full[s], 1);
            mbar_init(&bar_kv_empty[s], 1);
        }
        *abort_word = 0;
        fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, 512);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            tma_prefetch_desc(&tmap_q);
            tma_prefetch_desc(&tmap_k);
            tma_prefetch_desc(&tmap_v);
            const uint32_t k_bytes = static_cast<uint32_t>(k_chunks * kFaChunk);
            const uint32_t v_bytes = kVTrans ? static_cast<uint32_t>(2 * p.dv * 128) : static_cast<uint32_t>(v_chunks * kFaChunk);
            const int n_tiles = two_tiles ? 2 : 1;
            // Q tile 0, then K_0 so that the first MMA can start, then Q tile 1
            mbar_arrive_expect_tx(&bar_q_full[0], k_bytes);
            for (int c = 0; c < k_chunks; ++c) tma_load_3d(s_q + c * kFaChunk, &tmap_q, &bar_q_full[0], c * 64, q0, bh);
            bool q1_sent = false;
            for (int e = 0; e < 2 * n_blocks; ++e) {
                const int stage = e % kFaStages;
                const uint32_t phase = static_cast<uint32_t>((e / kFaStages) & 1);
                const int j = e >> 1;
                if (!mbar_wait(&bar_kv_empty[stage], phase ^ 1u, abort_word, kDevTimeoutProducer)) break;
                uint8_t* dst = s_kv + stage * kFaTile;
                if ((e & 1) == 0) {
                    mbar_arrive_expect_tx(&bar_kv_full[stage], k_bytes);
                    for (int c = 0; c < k_chunks; ++c)
                        tma_load_3d(dst + c * kFaChunk, &tmap_k, &bar_kv_full[stage], c * 64, j * kFaBN, bh);
                } else {
                    mbar_arrive_expect_tx(&bar_kv_full[stage], v_bytes);
                    if (kVTrans) {
                        for (int c = 0; c < 2; ++c)
                            tma_load_3d(dst + c * (p.dv * 128), &tmap_v, &bar_kv_full[stage], j * kFaBN + c * 64, 0, bh);
                    } else {
                        for (int c = 0; c < v_chunks; ++c)
                            tma_load_3d(dst + c * kFaChunk, &tmap_v, &bar_kv_full[stage], c * 64, j * kFaBN, bh);
                    }
                }
                if (!q1_sent && n_tiles == 2) {
                    mbar_arrive_expect_tx(&bar_q_full[1], k_bytes);
                    for (int c = 0; c < k_chunks; ++c)
                        tma_load_3d(s_q + kFaTile + c * kFaChunk, &tmap_q, &bar_q_full[1], c * 64, q0 + kFaBM, bh);
                    q1_sent = true;
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            const uint32_t idesc_s = make_idesc_f16_f32(kFaBM, kFaBN, false, false);
            const uint32_t idesc_o = make_idesc_f16_f32(kFaBM, p.dv, false, !kVTrans);
            const int n_tiles = two_tiles ? 2 : 1;

            auto kv_stage = [](int e) { return e % kFaStages; };
            auto kv_phase = [](int e) { return static_cast<uint32_t>((e / kFaStages) & 1); };

            // S_t = Q_t K_j^T
            auto issue_s = [&](int t, int j) {
                const uint32_t q_addr = smem_u32(s_q + t * kFaTile);
                const uint32_t k_addr = smem_u32(s_kv + kv_stage(2 * j) * kFaTile);
                const uint32_t d = tmem_base + static_cast<uint32_t>(t * kFaBN);
                for (int kk = 0; kk < k_steps; ++kk) {
                    const uint32_t off = static_cast<uint32_t>((kk >> 2) * kFaChunk + (kk & 3) * 32);
                    umma_f16_ss(d, make_smem_desc_sw128(q_addr + off, 16, 1024), make_smem_desc_sw128(k_addr + off, 16, 1024),
                                idesc_s, kk != 0);
                }
                umma_commit(&bar_s_full[t]);
            };
            // O_t += P_t V_j, P_t read from TMEM columns [t*128, t*128 + 64)
            auto issue_pv = [&](int t, int j) {
                const uint32_t v_addr = smem_u32(s_kv + kv_stage(2 * j + 1) * kFaTile);
                const uint32_t d = tmem_base + static_cast<uint32_t>(256 + t * 128);
                const uint32_t a = tmem_base + static_cast<uint32_t>(t * kFaBN);
                for (int kk = 0; kk < kFaBN / 16; ++kk) {
                    uint64_t b_desc;
                    if (kVTrans) {
                        const uint32_t b_off = static_cast<uint32_t>((kk >> 2) * (p.dv * 128) + (kk & 3) * 32);
                        b_desc = make_smem_desc_sw128(v_addr + b_off, 16, 1024);
                    } else {
                        b_desc = make_smem_desc_sw128(v_addr + static_cast<uint32_t>(kk * 2048), kFaChunk, 1024);
                    }
                    umma_f16_ts(d, a + static_cast<uint32_t>(kk * 8), b_desc, idesc_o, (j | kk) != 0);
                }
            };

            bool ok = mbar_wait(&bar_q_full[0], 0, abort_word, kDevTimeoutMma) &&
                      mbar_wait(&bar_kv_full[kv_stage(0)], kv_phase(0), abort_word, kDevTimeoutMma);
            if (ok) {
                tc_fence_after_sync();
                issue_s(0, 0);
                if (n_tiles == 2) {
                    ok = mbar_wait(&bar_q_full[1], 0, abort_word, kDevTimeoutMma);
                    if (ok) {
                        tc_fence_after_sync();
                        issue_s(1, 0);
                    }
                }
                umma_commit(&bar_kv_empty[kv_stage(0)]);
            }
            for (int j = 0; ok && j < n_blocks; ++j) {
                const bool has_next = j + 1 < n_blocks;
                if (!mbar_wait(&bar_kv_full[kv_stage(2 * j + 1)], kv_phase(2 * j + 1), abort_word, kDevTimeoutMma)) break;
                for (int t = 0; t < n_tiles; ++t) {
                    if (!mbar_wait(&bar_p_full[t], static_cast<uint32_t>(j & 1), abort_word, kDevTimeoutMma)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    issue_pv(t, j);
                    if (t == n_tiles - 1) umma_commit(&bar_kv_empty[kv_stage(2 * j + 1)]);
                    if (has_next) {
                        if (t == 0 &&
                            !mbar_wait(&bar_kv_full[kv_stage(2 * j + 2)], kv_phase(2 * j + 2), abort_word, kDevTimeoutMma)) {
                            ok = false;
                            break;
                        }
                        tc_fence_after_sync();
                        issue_s(t, j + 1);
                        if (t == n_tiles - 1) umma_commit(&bar_kv_empty[kv_stage(2 * j + 2)]);
                    } else {
                        umma_commit(&bar_o_full[t]);
                    }
                }
            }
        }
        __syncwarp();
    } else {
        // ---------------- softmax warpgroups: one thread per query row ----------------
        const int t = (warp - 2) >> 2;   // tile of this warpgroup
        const int quarter = warp & 3;
        const int row = q0 + t * kFaBM + quarter * 32 + lane;
        const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
        const uint32_t s_addr = tmem_base + lane_base + static_cast<uint32_t>(t * kFaBN);
        const uint32_t o_addr = tmem_base + lane_base + static_cast<uint32_t>(256 + t * 128);
        const float sc = p.scale_log2;
        float m_used = -INFINITY;
        float l_sum = 0.f;
        bool ok = (t == 0) || two_tiles;

        for (int j = 0; ok && j < n_blocks; ++j) {
            if (!mbar_wait_warp(&bar_s_full[t], static_cast<uint32_t>(j & 1), abort_word, kDevTimeoutSoftmax)) {
                ok = false;
                break;
            }
            tc_fence_after_sync();
            const int n_valid = min(kFaBN, p.seq_kv - j * kFaBN);

            // all 128 scores of this row into registers (one round trip to TMEM)
            uint32_t s[128];
            tmem_ld_x32(s_addr, *reinterpret_cast<uint32_t(*)[32]>(&s[0]));
            tmem_ld_x32(s_addr + 32, *reinterpret_cast<uint32_t(*)[32]>(&s[32]));
            tmem_ld_x32(s_addr + 64, *reinterpret_cast<uint32_t(*)[32]>(&s[64]));
            tmem_ld_x32(s_addr + 96, *reinterpret_cast<uint32_t(*)[32]>(&s[96]));
            tmem_ld_wait();
            if (n_valid < kFaBN) {
                const float masked = sc >= 0.f ? -INFINITY : INFINITY;  // scale * masked = -inf
#pragma unroll
                for (int i = 0; i < 128; ++i)
                    if (i >= n_valid) s[i] = __float_as_uint(masked);
            }
            // row maximum of scale * s: the extreme of the raw scores times the scale
            float e0 = __uint_as_float(s[0]), e1 = __uint_as_float(s[1]), e2 = __uint_as_float(s[2]), e3 = __uint_as_float(s[3]);
            if (sc >= 0.f) {
#pragma unroll
                for (int i = 4; i < 128; i += 4) {
                    e0 = fmaxf(e0, __uint_as_float(s[i]));
                    e1 = fmaxf(e1, __uint_as_float(s[i + 1]));
                    e2 = fmaxf(e2, __uint_as_float(s[i + 2]));
                    e3 = fmaxf(e3, __uint_as_float(s[i + 3]));
                }
                e0 = fmaxf(fmaxf(e0, e1), fmaxf(e2, e3));
            } else {
#pragma unroll
                for (int i = 4; i < 128; i += 4) {
                    e0 = fminf(e0, __uint_as_float(s[i]));
                    e1 = fminf(e1, __uint_as_float(s[i + 1]));
                    e2 = fminf(e2, __uint_as_float(s[i + 2]));
                    e3 = fminf(e3, __uint_as_float(s[i + 3]));
                }
                e0 = fminf(fminf(e0, e1), fminf(e2, e3));
            }
            const float mx = e0 * sc;
            float factor = 1.f;
            if (j == 0) {
                m_used = mx;
            } else if (mx > m_used + kFaRescaleThreshold) {
                factor = fast_exp2(m_used - mx);
                m_used = mx;
            }
            // s_full of block j was committed after P_t(j-1) V_{j-1}: O_t is quiescent here
            l_sum *= factor;
            if (__any_sync(0xffffffffu, factor != 1.f)) {
#pragma unroll 1
                for (int c = 0; c < p.dv / 16; ++c) {
                    uint32_t r[16];
                    tmem_ld_x16(o_addr + static_cast<uint32_t>(c * 16), r);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 16; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * factor);
                    tmem_st_x16(o_addr + static_cast<uint32_t>(c * 16), r);
                }
            }
            // exponentials, row sum, fp16 P written over the low half of the score columns
            const float neg_m = -m_used;
            float sum0 = 0.f, sum1 = 0.f, sum2 = 0.f, sum3 = 0.f;
#pragma unroll
            for (int i = 0; i < 64; i += 2) {
                const float a = fast_exp2(fmaf(__uint_as_float(s[2 * i]), sc, neg_m));
                const float b = fast_exp2(fmaf(__uint_as_float(s[2 * i + 1]), sc, neg_m));
                const float c2 = fast_exp2(fmaf(__uint_as_float(s[2 * i + 2]), sc, neg_m));
                const float d2 = fast_exp2(fmaf(__uint_as_float(s[2 * i + 3]), sc, neg_m));
                sum0 += a;
                sum1 += b;
                sum2 += c2;
                sum3 += d2;
                s[i] = pack_half2(a, b);
                s[i + 1] = pack_half2(c2, d2);
            }
            tmem_st_x32(s_addr, *reinterpret_cast<uint32_t(*)[32]>(&s[0]));
            tmem_st_x32(s_addr + 32, *reinterpret_cast<uint32_t(*)[32]>(&s[32]));
            const float sum01 = (sum0 + sum1) + (sum2 + sum3);
            l_sum += sum01;
            tmem_st_wait();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bar_p_full[t]);
        }

        // ---------------- epilogue ----------------
        if (ok && mbar_wait_warp(&bar_o_full[t], 0, abort_word, kDevTimeoutEpilogue)) {
            tc_fence_after_sync();
            const float inv_l = 1.f / l_sum;
            const int64_t out_row = static_cast<int64_t>(bh) * p.seq_q + row;
#pragma unroll 1
            for (int c = 0; c < p.dv / 16; ++c) {
                uint32_t r[16];
                tmem_ld_x16(o_addr + static_cast<uint32_t>(c * 16), r);
                tmem_ld_wait();
                if (row < p.seq_q) {
                    uint32_t h[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i)
                        h[i] = pack_half2(__uint_as_float(r[2 * i]) * inv_l, __uint_as_float(r[2 * i + 1]) * inv_l);
                    uint4* dst = reinterpret_cast<uint4*>(p.out + out_row * p.dv + c * 16);
                    dst[0] = make_uint4(h[0], h[1], h[2], h[3]);
                    dst[1] = make_uint4(h[4], h[5], h[6], h[7]);
                }
            }
            if (p.lse != nullptr && row < p.seq_q) p.lse[out_row] = (m_used + log2f(l_sum)) * 0.6931471805599453f;
        }
    }

    // ---------------- teardown ----------------
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, 512);
    }
    if (threadIdx.x == 0 && *abort_word != 0) atomicMax(p.status, *abort_word);
}

static int encode_attn_3d(CUtensorMap* out, const void* base, int64_t batch, int64_t rows, int64_t cols, uint32_t box_rows) {
    const uint64_t dims[3] = {static_cast<uint64_t>(cols), static_cast<uint64_t>(rows), static_cast<uint64_t>(batch)};
    const uint64_t strides[2] = {static_cast<uint64_t>(cols) * 2, static_cast<uint64_t>(rows) * static_cast<uint64_t>(cols) * 2};
    const uint32_t box[3] = {64, box_rows, 1};
    return encode_tmap_f16_sw128(out, base, 3, dims, strides, box);
}

// Launcher used by tc_flash_attn_fwd_f16 for seq_q > 128. Arguments are validated by the caller.
int launch_attn_pingpong(const void* Q, const void* K, const void* V, void* O, float* lse, int64_t bh, int64_t seq_q,
                         int64_t seq_kv, int64_t dk, int64_t dv, float scale, bool v_trans, cudaStream_t stream) {
    const DeviceInfo* dev = nullptr;
    if (int rc = current_device(&dev)) return rc;
    CUtensorMap tq, tk, tv;
    if (int rc = encode_attn_3d(&tq, Q, bh, seq_q, dk, kFaBM)) return rc;
    if (int rc = encode_attn_3d(&tk, K, bh, seq_kv, dk, kFaBN)) return rc;
    if (v_trans) {
        if (int rc = encode_attn_3d(&tv, V, bh, dv, seq_kv, static_cast<uint32_t>(dv))) return rc;
    } else {
        if (int rc = encode_attn_3d(&tv, V, bh, seq_kv, dv, kFaBN)) return rc;
    }
    AttnParams p;
    p.seq_q = static_cast<int>(seq_q);
    p.seq_kv = static_cast<int>(seq_kv);
    p.dk = static_cast<int>(dk);
    p.dv = static_cast<int>(dv);
    p.scale_log2 = scale * 1.4426950408889634f;
    p.out = static_cast<__half*>(O);
    p.lse = lse;
    p.status = dev->status_word;
    const dim3 grid(static_cast<unsigned>((seq_q + 2 * kFaBM - 1) / (2 * kFaBM)), static_cast<unsigned>(bh));
    static bool configured[2][64] = {};
    if (v_trans) {
        if (!configured[1][dev->device]) {
            TCB_CUDA(cudaFuncSetAttribute(attn_fwd_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kFaSmem));
            configured[1][dev->device] = true;
        }
        attn_fwd_kernel<true><<<grid, kFaThreads, kFaSmem, stream>>>(tq, tk, tv, p);
    } else {
        if (!configured[0][dev->device]) {
            TCB_CUDA(cudaFuncSetAttribute(attn_fwd_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kFaSmem));
            configured[0][dev->device] = true;
        }
        attn_fwd_kernel<false><<<grid, kFaThreads, kFaSmem, stream>>>(tq, tk, tv, p);
    }
    TCB_CUDA(cudaGetLastError());
    return TC_OK;
}

}  // namespace tcb
