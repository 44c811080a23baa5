// FlashAttention-2 forward for sequences longer than one tile: two 128-row Q tiles per CTA.
//
//   warp 0       TMA producer: both Q tiles once, then K_0, V_0, K_1, V_1, ... (128 KV rows each) through
//                one 4-stage ring;
//   warps 1, 2   tcgen05.mma issuers, one per Q tile (their instruction streams touch disjoint TMEM, so no
//                order is needed between them). Scores are produced and consumed in half blocks of 64 KV
//                rows; each tile owns two 64-column score buffers in TMEM. For half block g the issuer of tile t issues
//                O_t += P_t(g) V(g) (A operand read from TMEM) and then S_t(g+2) = Q_t K(g+2)^T into the
//                buffer P_t(g) just vacated, so the scores of the next half block are ready while the
//                softmax warps still work on the current one. The whole warp runs the loop, one elected lane
//                executes the MMAs; the loop holds one barrier wait and one commit per half block;
//   warp 3       forwarder: adds "the K / V tiles this step needs have landed" to the barrier the issuers wait on
//                anyway (P of half block g written), so that the issuers wait for nothing else;
//   warps 4..7   softmax warpgroup of tile 0, warps 8..11 of tile 1: one thread per query row. tcgen05.ld
//                64 fp32 scores, online softmax with fp32 running maximum and sum (exp2, scale folded
//                in), round to fp16 and tcgen05.st P over the columns the scores came from: P never
//                leaves TMEM. O_t stays in TMEM, is rescaled only when the row maximum grew by more
//                than 2^8 (after waiting for the PV product in flight), and is normalised once at the end.
//                These warps also hand the ring stages back to the producer: the MMAs of a CTA complete in
//                issue order, so seeing the scores of half block g means every older MMA has read its operands.
// TMEM: S_0a S_0b | S_1a S_1b | O_0 | O_1 (64, 64, 64, 64, 128, 128 columns). tcgen05.mma instructions
// of one CTA execute in issue order, so S_t(g+2) may overwrite P_t(g) right after P_t(g) V(g) was issued.
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
constexpr int kFaThreads = 384;
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
    int heads;
    int causal;          // 1: query row i sees KV rows j <= i + causal_off
    int causal_off;      // seq_kv - seq_q: the last query row sees every KV row
    int64_t out_stride_b;  // element strides of O over batch, head and query row
    int64_t out_stride_h;
    int64_t out_stride_s;
    __half* out;
    float* lse;
    uint32_t* status;
};

struct SoftmaxState {
    float m;   // reference maximum of the row (in units of log2, scale folded in)
    float l;   // sum of the row's exponentials against that reference
    bool ok;
};

// One half block of one query row per thread, the general way: the first half block of a tile (no reference yet),
// half blocks with masked columns (end of the sequence, causal diagonal), and half blocks in which some row of the
// warp outgrew its reference by more than 2^8. Whole warps call it. Reads the 64 scores at s_addr, raises the
// reference where needed (then O is rescaled, after `bar_pv` says that no product into it is in flight), writes the
// fp16 probabilities over the scores and returns the updated row state. Not inlined: it holds its own copy of the
// exponentials and is kept out of the loop that runs for every other half block.
static __device__ __noinline__ SoftmaxState softmax_half_block_general(uint32_t s_addr, uint32_t o_addr, int n_valid, float sc,
                                                                       int o_chunks, bool first, uint64_t* bar_pv,
                                                                       uint32_t bar_pv_parity, volatile uint32_t* abort_word,
                                                                       float m_used, float l_sum) {
    uint32_t s[64];
    tmem_ld_x32(s_addr, *reinterpret_cast<uint32_t(*)[32]>(&s[0]));
    tmem_ld_x32(s_addr + 32, *reinterpret_cast<uint32_t(*)[32]>(&s[32]));
    tmem_ld_wait();
    // scaled scores, masked columns at -inf (after scaling, so that a scale of zero masks too)
    float row_max = -INFINITY;
#pragma unroll
    for (int i = 0; i < 64; ++i) {
        const float x = i < n_valid ? __uint_as_float(s[i]) * sc : -INFINITY;
        s[i] = __float_as_uint(x);
        row_max = fmaxf(row_max, x);
    }
    float factor = 1.f;
    bool raised = false;
    if (first) {
        m_used = fmaxf(row_max, -1e30f);   // finite even for a row that sees no KV row at all
    } else if (row_max - m_used > kFaRescaleThreshold) {
        factor = fast_exp2(m_used - row_max);
        m_used = row_max;
        raised = true;
    }
    bool ok = true;
    if (__any_sync(0xffffffffu, raised)) {
        l_sum *= factor;
        ok = mbar_wait_warp(bar_pv, bar_pv_parity, abort_word, kDevTimeoutSoftmax);
        if (ok) {
            tc_fence_after_sync();
#pragma unroll 1
            for (int c = 0; c < o_chunks; ++c) {
                uint32_t r[16];
                tmem_ld_x16(o_addr + static_cast<uint32_t>(c * 16), r);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 16; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * factor);
                tmem_st_x16(o_addr + static_cast<uint32_t>(c * 16), r);
            }
        }
    }
    if (ok) {
        uint32_t pk[32];
        float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            const float a = fast_exp2(__uint_as_float(s[2 * i]) - m_used);
            const float b = fast_exp2(__uint_as_float(s[2 * i + 1]) - m_used);
            sum0 += a;
            sum1 += b;
            pk[i] = pack_half2(a, b);
        }
        tmem_st_x32(s_addr, pk);
        l_sum += sum0 + sum1;
        tmem_st_wait();
    }
    return SoftmaxState{m_used, l_sum, ok};
}

template <bool kVTrans>
__global__ void __launch_bounds__(kFaThreads, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_o, const AttnParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = align_smem_1024(smem_raw);
    uint8_t* s_q = smem;                   // two Q tiles
    uint8_t* s_kv = smem + 2 * kFaTile;    // ring of K / V tiles
    uint64_t* bars = reinterpret_cast<uint64_t*>(s_kv + kFaStages * kFaTile);
    uint64_t* bar_q_full = bars;                        // 2
    uint64_t* bar_kv_full = bars + 2;                   // kFaStages
    uint64_t* bar_kv_empty = bar_kv_full + kFaStages;   // kFaStages
    uint64_t* bar_s_full = bar_kv_empty + kFaStages;    // [tile][buffer]: 4
    uint64_t* bar_p_full = bar_s_full + 4;              // [tile][buffer]: 4
    uint64_t* bar_pv_done = bar_p_full + 4;             // [tile]: 2
    uint64_t* bar_o_full = bar_pv_done + 2;             // [tile]: 2
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_o_full + 2);
    volatile uint32_t* abort_word = tmem_slot + 1;

    // broadcast from lane 0, so that the compiler knows the role of a warp to be the same for all its lanes
    const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0);
    const int lane = threadIdx.x & 31;
    // with a causal mask the CTAs with the most KV blocks are scheduled first
    const int q_blk = p.causal ? static_cast<int>(gridDim.x - 1 - blockIdx.x) : static_cast<int>(blockIdx.x);
    const int q0 = q_blk * (2 * kFaBM);
    const int bh = blockIdx.y;
    const int head = bh % p.heads;
    const int bat = bh / p.heads;
    // KV rows this CTA needs: all of them, or up to the diagonal of its last query row
    const int kv_len = p.causal ? max(0, min(p.seq_kv, min(p.seq_q, q0 + 2 * kFaBM) + p.causal_off)) : p.seq_kv;
    const int n_halves = max(1, (kv_len + 63) / 64);       // 64-row half blocks (score granularity)
    const int n_blocks = (n_halves + 1) / 2;               // 128-row K / V blocks (TMA granularity)
    const int k_chunks = (p.dk + 63) / 64;
    const int v_chunks = (p.dv + 63) / 64;
    const int k_steps = p.dk / 16;
    const bool two_tiles = q0 + kFaBM < p.seq_q;  // the second tile may lie wholly outside the sequence

    if (threadIdx.x == 0) {
        for (int t = 0; t < 2; ++t) {
            mbar_init(&bar_q_full[t], 1);
            mbar_init(&bar_pv_done[t], 1);
            mbar_init(&bar_o_full[t], 1);
        }
        for (int i = 0; i < 4; ++i) {
            mbar_init(&bar_s_full[i], 1);
            mbar_init(&bar_p_full[i], 5);   // four softmax warps and the forwarder (warp 3)
        }
        for (int s = 0; s < kFaStages; ++s) {
            mbar_init(&bar_kv_full[s], 1);
            mbar_init(&bar_kv_empty[s], two_tiles ? 2 : 1);  // one release per tile in use (its softmax warpgroup)
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
            for (int c = 0; c < k_chunks; ++c) tma_load_4d(s_q + c * kFaChunk, &tmap_q, &bar_q_full[0], c * 64, q0, head, bat);
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
                        tma_load_4d(dst + c * kFaChunk, &tmap_k, &bar_kv_full[stage], c * 64, j * kFaBN, head, bat);
                } else {
                    mbar_arrive_expect_tx(&bar_kv_full[stage], v_bytes);
                    if (kVTrans) {
                        for (int c = 0; c < 2; ++c)
                            tma_load_4d(dst + c * (p.dv * 128), &tmap_v, &bar_kv_full[stage], j * kFaBN + c * 64, 0, head, bat);
                    } else {
                        for (int c = 0; c < v_chunks; ++c)
                            tma_load_4d(dst + c * kFaChunk, &tmap_v, &bar_kv_full[stage], c * 64, j * kFaBN, head, bat);
                    }
                }
                if (!q1_sent && n_tiles == 2) {
                    mbar_arrive_expect_tx(&bar_q_full[1], k_bytes);
                    for (int c = 0; c < k_chunks; ++c)
                        tma_load_4d(s_q + kFaTile + c * kFaChunk, &tmap_q, &bar_q_full[1], c * 64, q0 + kFaBM, head, bat);
                    q1_sent = true;
                }
            }
        }
        __syncwarp();
    } else if (warp == 1 || warp == 2) {
        // ---------------- MMA issuers: warp 1 drives tile 0, warp 2 drives tile 1 ----------------
        // The whole warp runs the role and one elected lane executes the MMAs and their commits (a commit tracks the
        // MMAs of the thread that executes it). With every lane on the same path the descriptor arithmetic stays in
        // the uniform datapath, whose registers tcgen05.mma reads; behind a branch on the lane index every operand
        // would first be moved there, which costs a fifth of the tensor pipe's time at these MMA sizes (measured:
        // 1143 against 1261 cycles for the 24 MMAs of a half block of both tiles).
        const int t = warp - 1;
        if (t == 0 || two_tiles) {
            const bool leader = elect_one_sync();
            const uint32_t idesc_s = make_idesc_f16_f32(kFaBM, 64, false, false);
            const uint32_t idesc_o = make_idesc_f16_f32(kFaBM, p.dv, false, !kVTrans);

            auto kv_stage = [](int e) { return e % kFaStages; };
            auto kv_phase = [](int e) { return static_cast<uint32_t>((e / kFaStages) & 1); };

            const uint32_t desc_hi = smem_desc_hi_sw128(1024);
            constexpr uint32_t kTileStep = static_cast<uint32_t>(kFaTile) >> 4;  // descriptor address units per tile
            const uint32_t q_lo = smem_desc_lo(smem_u32(s_q), 16) + static_cast<uint32_t>(t) * kTileStep;
            const uint32_t kv_lo0 = smem_desc_lo(smem_u32(s_kv), 16);
            const uint32_t v_lbo_word = kVTrans ? 0u : ((static_cast<uint32_t>(kFaChunk) >> 4) - 1u) << 16;  // LBO 16 -> kFaChunk
            const uint32_t v_half_step = kVTrans ? static_cast<uint32_t>(p.dv * 128) >> 4 : (64u * 128u) >> 4;
            const uint32_t v_k_step = kVTrans ? 2u : 2048u >> 4;
            const uint32_t tmem_s = tmem_base + static_cast<uint32_t>(t * 128);
            const uint32_t tmem_o = tmem_base + static_cast<uint32_t>(256 + t * 128);

            // S_t(g) = Q_t K(g)^T for the 64 KV rows of half block g, into score buffer g & 1
            auto issue_s = [&](int g) {
                const int h = g & 1;
                const uint32_t b_lo = kv_lo0 + static_cast<uint32_t>(kv_stage(2 * (g >> 1))) * kTileStep + static_cast<uint32_t>(h * ((64 * 128) >> 4));
                const uint32_t d = tmem_s + static_cast<uint32_t>(h * 64);
#pragma unroll
                for (int kk = 0; kk < 8; ++kk) {
                    if (kk < k_steps) {
                        const uint32_t off = static_cast<uint32_t>(((kk >> 2) * kFaChunk + (kk & 3) * 32) >> 4);
                        if (leader)
                            umma_f16_ss(d, smem_desc_join(q_lo + off, desc_hi), smem_desc_join(b_lo + off, desc_hi), idesc_s, kk != 0);
                    }
                }
                if (leader) umma_commit(&bar_s_full[t * 2 + h]);
            };
            // O_t += P_t(g) V(g); P_t(g) is read from the first 32 columns of score buffer g & 1
            auto issue_pv = [&](int g) {
                const int h = g & 1;
                const uint32_t b_lo = kv_lo0 + static_cast<uint32_t>(kv_stage(2 * (g >> 1) + 1)) * kTileStep + v_lbo_word +
                                      static_cast<uint32_t>(h) * v_half_step;
                const uint32_t a = tmem_s + static_cast<uint32_t>(h * 64);
#pragma unroll
                for (int kk = 0; kk < 4; ++kk) {
                    if (leader)
                        umma_f16_ts(tmem_o, a + static_cast<uint32_t>(kk * 8),
                                    smem_desc_join(b_lo + static_cast<uint32_t>(kk) * v_k_step, desc_hi), idesc_o, (g | kk) != 0);
                }
            };

            // prologue: the first two half blocks of scores (both from K_0)
            bool ok = mbar_wait_warp(&bar_q_full[t], 0, abort_word, kDevTimeoutMma) &&
                      mbar_wait_warp(&bar_kv_full[kv_stage(0)], kv_phase(0), abort_word, kDevTimeoutMma);
            if (ok) {
                tc_fence_after_sync();
                issue_s(0);
                if (n_halves > 1) issue_s(1);
            }
            // Every barrier operation between two MMAs of this thread is a bubble in the tensor pipe, whose queue runs
            // barely an MMA or two behind the issuing thread (measured: 30 to 65 cycles per commit, 55 per wait that
            // succeeds at once). So the loop holds one wait and one commit per half block: p_full also stands for "the
            // K / V tiles of this step have landed" (warp 3 forwards that), the ring stages are released by the softmax
            // warps when they see the scores that were issued behind the last MMA reading a stage, and the completion of
            // a P V product is read off the scores issued behind it.
            for (int g = 0; ok && g < n_halves; ++g) {
                const bool more_s = g + 2 < n_halves;
                if (!mbar_wait_warp(&bar_p_full[t * 2 + (g & 1)], static_cast<uint32_t>((g >> 1) & 1), abort_word, kDevTimeoutMma)) break;
                tc_fence_after_sync();
                issue_pv(g);
                if (more_s) issue_s(g + 2);   // commits to s_full
                if (leader && g == n_halves - 2) umma_commit(&bar_pv_done[t]);   // no scores follow this product
                if (leader && g == n_halves - 1) umma_commit(&bar_o_full[t]);
            }
        }
        __syncwarp();
    } else if (warp == 3) {
        // ---------------- forwarder ----------------
        // Adds "the tiles the issuers need at half block g have landed" to p_full of half block g as its fifth arrival:
        // V of block g / 2 for P(g) V and K of block (g + 2) / 2 for the scores of half block g + 2, both new at even g.
        // An arrival counts for the barrier's current phase, so the one for g waits until the phase of g - 2 is complete.
        if (lane == 0) {
            auto kv_stage = [](int e) { return e % kFaStages; };
            auto kv_phase = [](int e) { return static_cast<uint32_t>((e / kFaStages) & 1); };
            const int n_tiles = two_tiles ? 2 : 1;
            bool ok = true;
            for (int g = 0; ok && g < n_halves; ++g) {
                if ((g & 1) == 0) {
                    const int j = g >> 1;
                    ok = mbar_wait(&bar_kv_full[kv_stage(2 * j + 1)], kv_phase(2 * j + 1), abort_word, kDevTimeoutMma) &&
                         (g + 2 >= n_halves ||
                          mbar_wait(&bar_kv_full[kv_stage(2 * j + 2)], kv_phase(2 * j + 2), abort_word, kDevTimeoutMma));
                }
                for (int t = 0; ok && t < n_tiles; ++t) {
                    if (g >= 2)
                        ok = mbar_wait(&bar_p_full[t * 2 + (g & 1)], static_cast<uint32_t>(((g - 2) >> 1) & 1), abort_word, kDevTimeoutMma);
                    if (ok) mbar_arrive(&bar_p_full[t * 2 + (g & 1)]);
                }
            }
        }
        __syncwarp();
    } else {
        // ---------------- softmax warpgroups: one thread per query row ----------------
        const int t = (warp - 4) >> 2;   // tile of this warpgroup
        const int quarter = warp & 3;
        const int row = q0 + t * kFaBM + quarter * 32 + lane;
        const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
        const uint32_t s_base = tmem_base + lane_base + static_cast<uint32_t>(t * 128);
        const uint32_t o_addr = tmem_base + lane_base + static_cast<uint32_t>(256 + t * 128);
        const float sc = p.scale_log2;
        float m_used = -INFINITY;
        float l_sum = 0.f;
        bool ok = (t == 0) || two_tiles;
        for (int g = 0; ok && g < n_halves; ++g) {
            const int h = g & 1;
            if (!mbar_wait_warp(&bar_s_full[t * 2 + h], static_cast<uint32_t>((g >> 1) & 1), abort_word, kDevTimeoutSoftmax)) {
                ok = false;
                break;
            }
            tc_fence_after_sync();
            // The MMAs of one CTA complete in issue order: scores of half block g complete mean that K of block g / 2 has
            // been read for this half, and that P(g-2) V, issued before them, has read its half of V.
            if (quarter == 0 && lane == 0) {
                if ((g & 1) == 1 || g == n_halves - 1) mbar_arrive(&bar_kv_empty[(2 * (g >> 1)) % kFaStages]);
                if ((g & 1) == 1 && g >= 3) mbar_arrive(&bar_kv_empty[(2 * ((g - 2) >> 1) + 1) % kFaStages]);
            }
            const uint32_t s_addr = s_base + static_cast<uint32_t>(h * 64);
            // columns of this half block the row may see: the end of the sequence and, with a causal mask, the diagonal
            int n_valid = min(64, p.seq_kv - g * 64);
            if (p.causal) n_valid = min(n_valid, row + p.causal_off + 1 - g * 64);

            // The common half block (not the first, no masked column in this warp) runs the short path below; everything
            // else goes through softmax_half_block_general, a function of its own, so that the loop the eight softmax
            // warps run 64 times per tile stays small in instruction memory.
            // What the general path waits for before it rescales O_t, which may still be the target of P_t(g-1) V(g-1): the
            // scores of half block g + 1 were issued behind that product (and do not depend on this half block), so their
            // completion is its completion; behind the product before the last one the issuer commits to pv_done instead.
            uint64_t* const bar_pv = g == n_halves - 1 ? &bar_pv_done[t] : &bar_s_full[t * 2 + ((g + 1) & 1)];
            const uint32_t bar_pv_parity = g == n_halves - 1 ? 0u : static_cast<uint32_t>(((g + 1) >> 1) & 1);
            bool general = g == 0 || __any_sync(0xffffffffu, n_valid < 64);
            if (!general) {
                // the 64 scores of this row and half block into registers
                uint32_t s[64];
                tmem_ld_x32(s_addr, *reinterpret_cast<uint32_t(*)[32]>(&s[0]));
                tmem_ld_x32(s_addr + 32, *reinterpret_cast<uint32_t(*)[32]>(&s[32]));
                tmem_ld_wait();
                // Exponentials are taken against the reference maximum m_used of the previous half blocks without looking
                // at this half block's maximum first. The reference has to be replaced when some row outgrew it by more
                // than 2^8, which after the first few half blocks is rare; no score exceeds it by that much if the 64
                // exponentials sum to 2^8 or less, so the sum (needed anyway) is the test, and a larger, infinite or
                // undefined one sends the half block through the general path, which looks at the maximum itself and
                // works from the scores still in TMEM. The arithmetic runs on packed pairs (half the FMA-pipe
                // instructions), and every fourth pair takes its exponentials on the FMA pipe as well (poly_exp2_pair),
                // which leaves the special-function unit three quarters of the work: measured 1288 TFLOP/s against
                // 1179 with scalar arithmetic and every exponential on that unit, 1237 with packed arithmetic alone,
                // 1259 with every second pair on the FMA pipe.
                uint32_t pk[32];
                const uint64_t sc2 = pack2(sc, sc), neg_m2 = pack2(-m_used, -m_used);
                uint64_t sum_a = pack2(0.f, 0.f), sum_b = sum_a;
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const uint64_t x2 = fma2(pack2(__uint_as_float(s[2 * i]), __uint_as_float(s[2 * i + 1])), sc2, neg_m2);
                    float xa, xb, a, b;
                    unpack2(x2, xa, xb);
                    if ((i & 3) == 3) {
                        poly_exp2_pair(xa, xb, a, b);
                    } else {
                        a = fast_exp2(xa);
                        b = fast_exp2(xb);
                    }
                    if (i & 1) sum_b = add2(sum_b, pack2(a, b)); else sum_a = add2(sum_a, pack2(a, b));
                    pk[i] = pack_half2(a, b);
                }
                float sum0, sum1, sum2, sum3;
                unpack2(sum_a, sum0, sum1);
                unpack2(sum_b, sum2, sum3);
                const float half_sum = (sum0 + sum1) + (sum2 + sum3);
                general = __any_sync(0xffffffffu, !(half_sum <= 256.f));
                if (!general) {
                    tmem_st_x32(s_addr, pk);
                    l_sum += half_sum;
                    tmem_st_wait();
                }
            }
            if (general) {
                const SoftmaxState st = softmax_half_block_general(s_addr, o_addr, n_valid, sc, p.dv / 16, g == 0, bar_pv, bar_pv_parity,
                                                                   abort_word, m_used, l_sum);
                m_used = st.m;
                l_sum = st.l;
                if (!st.ok) {
                    ok = false;
                    break;
                }
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bar_p_full[t * 2 + h]);
        }

        // ---------------- epilogue ----------------
        // The normalised rows go through shared memory and leave as TMA stores of whole 128-byte lines: the Q tile of
        // this warpgroup's tile has been read by its last score MMA long before the last P V product completes, so its
        // 32 KiB (128 rows x 256 bytes, the 128-byte-swizzled box layout of the output map) serve as staging. Rows and
        // columns outside the output are clipped by TMA.
        const bool o_ready = ok && mbar_wait_warp(&bar_o_full[t], 0, abort_word, kDevTimeoutEpilogue);
        if (o_ready) {
            tc_fence_after_sync();
            const float inv_l = l_sum > 0.f ? 1.f / l_sum : 0.f;   // a fully masked row yields zeros
            const int r_in_tile = quarter * 32 + lane;
            uint8_t* stage_row = s_q + t * kFaTile + r_in_tile * 128;
            int c = 0;
#pragma unroll 1
            // 64 columns per round trip to TMEM while they last (each trip costs its latency once), 16 for the rest
            for (; c + 4 <= p.dv / 16; c += 4) {
                uint32_t r[64];
                tmem_ld_x32(o_addr + static_cast<uint32_t>(c * 16), *reinterpret_cast<uint32_t(*)[32]>(&r[0]));
                tmem_ld_x32(o_addr + static_cast<uint32_t>(c * 16 + 32), *reinterpret_cast<uint32_t(*)[32]>(&r[32]));
                tmem_ld_wait();
                uint8_t* chunk = stage_row + (c >> 2) * kFaChunk;
#pragma unroll
                for (int cc = 0; cc < 4; ++cc) {
                    uint32_t h[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i)
                        h[i] = pack_half2(__uint_as_float(r[cc * 16 + 2 * i]) * inv_l, __uint_as_float(r[cc * 16 + 2 * i + 1]) * inv_l);
                    const int piece = cc * 2;
                    *reinterpret_cast<uint4*>(chunk + (((piece) ^ (r_in_tile & 7)) << 4)) = make_uint4(h[0], h[1], h[2], h[3]);
                    *reinterpret_cast<uint4*>(chunk + (((piece + 1) ^ (r_in_tile & 7)) << 4)) = make_uint4(h[4], h[5], h[6], h[7]);
                }
            }
#pragma unroll 1
            for (; c < p.dv / 16; ++c) {
                uint32_t r[16];
                tmem_ld_x16(o_addr + static_cast<uint32_t>(c * 16), r);
                tmem_ld_wait();
                uint32_t h[8];
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    h[i] = pack_half2(__uint_as_float(r[2 * i]) * inv_l, __uint_as_float(r[2 * i + 1]) * inv_l);
                uint8_t* chunk = stage_row + (c >> 2) * kFaChunk;      // 64 output columns per 16 KiB chunk
                const int piece = (c & 3) * 2;                           // 16-byte pieces of this row inside the chunk
                *reinterpret_cast<uint4*>(chunk + (((piece) ^ (r_in_tile & 7)) << 4)) = make_uint4(h[0], h[1], h[2], h[3]);
                *reinterpret_cast<uint4*>(chunk + (((piece + 1) ^ (r_in_tile & 7)) << 4)) = make_uint4(h[4], h[5], h[6], h[7]);
            }
            if (p.lse != nullptr && row < p.seq_q)
                p.lse[static_cast<int64_t>(bh) * p.seq_q + row] = (m_used + log2f(l_sum)) * 0.6931471805599453f;
            fence_proxy_async_smem();
        }
        // all four warps of the tile have staged their rows (or given up) before one thread hands the tile to TMA
        asm volatile("bar.sync %0, 128;" ::"r"(1 + t) : "memory");
        if (o_ready && quarter == 0 && lane == 0 && q0 + t * kFaBM < p.seq_q) {
            for (int c = 0; c < v_chunks; ++c)
                tma_store_4d(&tmap_o, s_q + t * kFaTile + c * kFaChunk, c * 64, q0 + t * kFaBM, head, bat);
            tma_store_commit();
            tma_store_wait_read<0>();   // the tile has left shared memory; the grid's completion covers the writes
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

// 4-D map over (column, row, head, batch) with element strides for row, head and batch.
static int encode_attn_4d(CUtensorMap* out, const void* base, int64_t batch, int64_t heads, int64_t rows, int64_t cols,
                          int64_t stride_row, int64_t stride_head, int64_t stride_batch, uint32_t box_rows) {
    const uint64_t dims[4] = {static_cast<uint64_t>(cols), static_cast<uint64_t>(rows), static_cast<uint64_t>(heads),
                              static_cast<uint64_t>(batch)};
    const uint64_t strides[3] = {static_cast<uint64_t>(stride_row) * 2, static_cast<uint64_t>(stride_head) * 2,
                                 static_cast<uint64_t>(stride_batch) * 2};
    const uint32_t box[4] = {64, box_rows, 1, 1};
    return encode_tmap_f16_sw128(out, base, 4, dims, strides, box);
}

// Launcher behind the attention entry points. Arguments are validated by the caller. seq_major: operands
// are [batch, seq, heads, dim] instead of [batch, heads, seq, dim] (not with a transposed V).
int launch_attn_pingpong(const void* Q, const void* K, const void* V, void* O, float* lse, int64_t batch, int64_t heads,
                         int64_t seq_q, int64_t seq_kv, int64_t dk, int64_t dv, float scale, bool v_trans, bool causal,
                         bool seq_major, cudaStream_t stream) {
    const DeviceInfo* dev = nullptr;
    if (int rc = current_device(&dev)) return rc;
    CUtensorMap tq, tk, tv;
    auto encode = [&](CUtensorMap* m, const void* base, int64_t rows, int64_t cols, uint32_t box_rows) {
        if (seq_major) return encode_attn_4d(m, base, batch, heads, rows, cols, heads * cols, cols, rows * heads * cols, box_rows);
        return encode_attn_4d(m, base, batch, heads, rows, cols, cols, rows * cols, heads * rows * cols, box_rows);
    };
    if (int rc = encode(&tq, Q, seq_q, dk, kFaBM)) return rc;
    if (int rc = encode(&tk, K, seq_kv, dk, kFaBN)) return rc;
    if (v_trans) {
        if (int rc = encode(&tv, V, dv, seq_kv, static_cast<uint32_t>(dv))) return rc;
    } else {
        if (int rc = encode(&tv, V, seq_kv, dv, kFaBN)) return rc;
    }
    AttnParams p;
    p.seq_q = static_cast<int>(seq_q);
    p.seq_kv = static_cast<int>(seq_kv);
    p.dk = static_cast<int>(dk);
    p.dv = static_cast<int>(dv);
    p.scale_log2 = scale * 1.4426950408889634f;
    p.heads = static_cast<int>(heads);
    p.causal = causal ? 1 : 0;
    p.causal_off = static_cast<int>(seq_kv - seq_q);
    p.out_stride_s = seq_major ? heads * dv : dv;
    p.out_stride_h = seq_major ? dv : seq_q * dv;
    p.out_stride_b = heads * seq_q * dv;
    p.out = static_cast<__half*>(O);
    p.lse = lse;
    p.status = dev->status_word;
    // the output as the input maps see their tensors: [batch, heads, seq_q, dv] or, sequence-major, [batch, seq_q, heads, dv]
    CUtensorMap to;
    if (int rc = encode(&to, O, seq_q, dv, kFaBM)) return rc;
    const dim3 grid(static_cast<unsigned>((seq_q + 2 * kFaBM - 1) / (2 * kFaBM)), static_cast<unsigned>(batch * heads));
    static OncePerDevice once[2];
    if (v_trans) {
        if (int rc = raise_smem_limit_once(once[1], dev->device, attn_fwd_kernel<true>, kFaSmem)) return rc;
        attn_fwd_kernel<true><<<grid, kFaThreads, kFaSmem, stream>>>(tq, tk, tv, to, p);
    } else {
        if (int rc = raise_smem_limit_once(once[0], dev->device, attn_fwd_kernel<false>, kFaSmem)) return rc;
        attn_fwd_kernel<false><<<grid, kFaThreads, kFaSmem, stream>>>(tq, tk, tv, to, p);
    }
    TCB_CUDA(cudaGetLastError());
    return TC_OK;
}

}  // namespace tcb
