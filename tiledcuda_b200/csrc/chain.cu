// Two chained contractions with the intermediate held on chip:
//   back-to-back GEMM      E = fp16(A B) D                     (kSoftmax = false, fp32 output)
//   FlashAttention-2 fwd   O = softmax(scale Q K^T) V          (kSoftmax = true,  fp16 output)
//
// One CTA owns 128 rows of the left operand of one batch entry (one (batch, head) for attention)
// and walks the inner dimension (N of the B2B GEMM, the KV sequence for attention) in blocks of 128:
//   warp 0      TMA producer: the Q/A tile once, then K/B and V/D blocks into two-stage rings;
//   warp 1      tcgen05.mma issuer: S = Q K_j^T into one of two TMEM buffers, then O += P_j V_j;
//               S of block j+1 is issued before P_j V_j so the tensor pipe works while the other
//               warps are busy with block j;
//   warps 2..5  one thread per row: tcgen05.ld S, (online softmax with fp32 running max and sum,
//               exp2 with the scale folded in), round to fp16, write P into 128-byte-swizzled
//               shared memory where it becomes operand A of the second MMA. The O accumulator
//               stays in TMEM for the whole walk; it is rescaled only when a row's maximum grows
//               by more than 2^8, and normalised once at the end.
// The intermediate S/P never touches HBM. V is taken either as [kv, dv] rows (an MN-major MMA
// operand) or transposed [dv, kv] (K-major), which is how the reference feeds it.
//
// Stands in for KeFusedGemm (examples/cpp/02_fused_two_gemms/fused_gemm.hpp:98-181) and
// flash_attention (src/kernels/flash_attn.cu:134-312); unlike the latter the statistics are fp32,
// Q is loaded once, and O is divided by the running sum once instead of once per KV block.
#include <math.h>

#include <string.h>

#include "host.h"
#include "sm100.cuh"

namespace tcb {

constexpr int kChBM = 128;       // rows per CTA
constexpr int kChBN = 128;       // inner block (kv rows / N columns) per step
constexpr int kChStages = 2;     // K and V ring depth
constexpr int kChThreads = 192;
constexpr int kChTile = 128 * 128 * 2;  // bytes of a 128 x 128 fp16 tile (two 64-wide swizzle chunks)
constexpr int kChChunk = 128 * 64 * 2;  // bytes of one 128 x 64 chunk
constexpr int kChSmem = kChTile * (2 + 2 * kChStages) + 256 + 1024;
constexpr float kRescaleThreshold = 8.0f;  // log2 units

struct ChainParams {
    int rows;        // seq_q / M
    int inner;       // seq_kv / N
    int dk;          // head_dim / K   (<= 128, multiple of 16)
    int dv;          // head_dim_v / P (<= 128, multiple of 16)
    float scale_log2;  // softmax scale * log2(e)
    void* out;       // fp16 [batch, rows, dv] (attention) or fp32 (B2B)
    float* lse;      // optional, attention only
    uint32_t* status;
    int store_by_tma;  // B2B: fp32 output through shared memory and TMA stores (tmap_o is valid)
};

template <bool kSoftmax, bool kVTrans>
__global__ void __launch_bounds__(kChThreads, 1)
chain_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
             const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_o, const ChainParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = align_smem_1024(smem_raw);
    uint8_t* s_q = smem;
    uint8_t* s_p = smem + kChTile;
    uint8_t* s_k = smem + 2 * kChTile;
    uint8_t* s_v = s_k + kChStages * kChTile;
    uint64_t* bars = reinterpret_cast<uint64_t*>(s_v + kChStages * kChTile);
    uint64_t* bar_q_full = bars;                    // 1
    uint64_t* bar_k_full = bars + 1;                // kChStages
    uint64_t* bar_k_empty = bar_k_full + kChStages;
    uint64_t* bar_v_full = bar_k_empty + kChStages;
    uint64_t* bar_v_empty = bar_v_full + kChStages;
    uint64_t* bar_s_full = bar_v_empty + kChStages;  // 2
    uint64_t* bar_s_empty = bar_s_full + 2;          // 2
    uint64_t* bar_p_full = bar_s_empty + 2;          // 1
    uint64_t* bar_p_empty = bar_p_full + 1;          // 1
    uint64_t* bar_o_full = bar_p_empty + 1;          // 1
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_o_full + 1);
    volatile uint32_t* abort_word = tmem_slot + 1;

    // broadcast from lane 0, so that the compiler knows the role of a warp to be the same for all its lanes
    const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0);
    const int lane = threadIdx.x & 31;
    const int q0 = blockIdx.x * kChBM;
    const int bh = blockIdx.y;
    const int n_blocks = (p.inner + kChBN - 1) / kChBN;
    const int k_chunks = (p.dk + 63) / 64;   // 64-wide swizzle chunks of the first contraction
    const int v_chunks = (p.dv + 63) / 64;   // 64-wide chunks of dv (V as [kv, dv])
    const int k_steps = p.dk / 16;

    if (threadIdx.x == 0) {
        mbar_init(bar_q_full, 1);
        for (int s = 0; s < kChStages; ++s) {
            mbar_init(&bar_k_full[s], 1);
            mbar_init(&bar_k_empty[s], 1);
            mbar_init(&bar_v_full[s], 1);
            mbar_init(&bar_v_empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&bar_s_full[b], 1);
            mbar_init(&bar_s_empty[b], 4);
        }
        mbar_init(bar_p_full, 4);
        mbar_init(bar_p_empty, 1);
        mbar_init(bar_o_full, 1);
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
    const uint32_t tmem_s0 = tmem_base;          // S buffers: columns [0,128) and [128,256)
    const uint32_t tmem_o = tmem_base + 256;     // O accumulator: columns [256, 256 + dv)
    // No global memory has been touched yet: a kernel queued behind this one may start its set-up on free SMs,
    // and this one waits for its predecessor only before its first load (producer) or store (row threads).
    grid_launch_dependents();

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        // Producer and MMA issuer run as whole warps; one elected lane executes the TMA, MMA and commit instructions.
        // With every lane on the same path the address and descriptor arithmetic stays in the uniform datapath, whose
        // registers those instructions read; behind a branch on the lane index every operand is moved there first.
        const bool leader = elect_one_sync();
        {
            if (leader) {
                tma_prefetch_desc(&tmap_q);
                tma_prefetch_desc(&tmap_k);
                tma_prefetch_desc(&tmap_v);
            }
            grid_dependency_wait();
            if (leader) {
                mbar_arrive_expect_tx(bar_q_full, static_cast<uint32_t>(k_chunks * kChChunk));
                for (int c = 0; c < k_chunks; ++c) tma_load_3d(s_q + c * kChChunk, &tmap_q, bar_q_full, c * 64, q0, bh);
            }
            const uint32_t v_bytes = kVTrans ? static_cast<uint32_t>(2 * p.dv * 128) : static_cast<uint32_t>(v_chunks * kChChunk);
            for (int j = 0; j < n_blocks; ++j) {
                const int stage = j % kChStages;
                const uint32_t phase = static_cast<uint32_t>((j / kChStages) & 1);
                if (!mbar_wait_warp(&bar_k_empty[stage], phase ^ 1u, abort_word, kDevTimeoutProducer)) break;
                if (leader) {
                    mbar_arrive_expect_tx(&bar_k_full[stage], static_cast<uint32_t>(k_chunks * kChChunk));
                    for (int c = 0; c < k_chunks; ++c)
                        tma_load_3d(s_k + stage * kChTile + c * kChChunk, &tmap_k, &bar_k_full[stage], c * 64, j * kChBN, bh);
                }
                if (!mbar_wait_warp(&bar_v_empty[stage], phase ^ 1u, abort_word, kDevTimeoutProducer)) break;
                if (leader) {
                    mbar_arrive_expect_tx(&bar_v_full[stage], v_bytes);
                    if (kVTrans) {
                        // V^T rows are dv, inner dimension is kv: two 64-wide kv chunks of dv rows each
                        for (int c = 0; c < 2; ++c)
                            tma_load_3d(s_v + stage * kChTile + c * (p.dv * 128), &tmap_v, &bar_v_full[stage],
                                        j * kChBN + c * 64, 0, bh);
                    } else {
                        for (int c = 0; c < v_chunks; ++c)
                            tma_load_3d(s_v + stage * kChTile + c * kChChunk, &tmap_v, &bar_v_full[stage], c * 64, j * kChBN, bh);
                    }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        const bool leader = elect_one_sync();
        {
            const uint32_t idesc_s = make_idesc_f16_f32(kChBM, kChBN, false, false);
            const uint32_t idesc_o = make_idesc_f16_f32(kChBM, p.dv, false, !kVTrans);
            bool ok = mbar_wait_warp(bar_q_full, 0, abort_word, kDevTimeoutMma);

            auto issue_s = [&](int j) -> bool {
                const int stage = j % kChStages;
                const uint32_t phase = static_cast<uint32_t>((j / kChStages) & 1);
                const int buf = j & 1;
                const uint32_t buf_phase = static_cast<uint32_t>((j >> 1) & 1);
                if (!mbar_wait_warp(&bar_k_full[stage], phase, abort_word, kDevTimeoutMma)) return false;
                if (!mbar_wait_warp(&bar_s_empty[buf], buf_phase ^ 1u, abort_word, kDevTimeoutMma)) return false;
                tc_fence_after_sync();
                const uint32_t q_addr = smem_u32(s_q);
                const uint32_t k_addr = smem_u32(s_k + stage * kChTile);
                for (int kk = 0; kk < k_steps; ++kk) {
                    const uint32_t off = static_cast<uint32_t>((kk >> 2) * kChChunk + (kk & 3) * 32);
                    if (leader)
                        umma_f16_ss(tmem_s0 + static_cast<uint32_t>(buf * kChBN), make_smem_desc_sw128(q_addr + off, 16, 1024),
                                    make_smem_desc_sw128(k_addr + off, 16, 1024), idesc_s, kk != 0);
                }
                if (leader) {
                    umma_commit(&bar_s_full[buf]);
                    umma_commit(&bar_k_empty[stage]);
                }
                return true;
            };

            if (ok) ok = issue_s(0);
            for (int j = 0; ok && j < n_blocks; ++j) {
                if (j + 1 < n_blocks) {
                    if (!issue_s(j + 1)) break;
                }
                const int stage = j % kChStages;
                const uint32_t phase = static_cast<uint32_t>((j / kChStages) & 1);
                if (!mbar_wait_warp(bar_p_full, static_cast<uint32_t>(j & 1), abort_word, kDevTimeoutMma)) break;
                if (!mbar_wait_warp(&bar_v_full[stage], phase, abort_word, kDevTimeoutMma)) break;
                tc_fence_after_sync();
                const uint32_t p_addr = smem_u32(s_p);
                const uint32_t v_addr = smem_u32(s_v + stage * kChTile);
                for (int kk = 0; kk < kChBN / 16; ++kk) {
                    const uint32_t a_off = static_cast<uint32_t>((kk >> 2) * kChChunk + (kk & 3) * 32);
                    uint64_t b_desc;
                    if (kVTrans) {
                        const uint32_t b_off = static_cast<uint32_t>((kk >> 2) * (p.dv * 128) + (kk & 3) * 32);
                        b_desc = make_smem_desc_sw128(v_addr + b_off, 16, 1024);
                    } else {
                        // MN-major: 16 kv rows of 128 bytes per step; dv chunks of 64 are kChChunk apart
                        b_desc = make_smem_desc_sw128(v_addr + static_cast<uint32_t>(kk * 2048), kChChunk, 1024);
                    }
                    if (leader) umma_f16_ss(tmem_o, make_smem_desc_sw128(p_addr + a_off, 16, 1024), b_desc, idesc_o, (j | kk) != 0);
                }
                if (leader) {
                    umma_commit(bar_p_empty);
                    umma_commit(&bar_v_empty[stage]);
                }
            }
            if (ok && leader) umma_commit(bar_o_full);
        }
        __syncwarp();
    } else {
        // ---------------- softmax / conversion / epilogue: one thread per row ----------------
        const int quarter = warp & 3;
        const int row_in_tile = quarter * 32 + lane;
        const int row = q0 + row_in_tile;
        const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
        float m_used = -INFINITY;  // running maximum the exponentials are taken against (log2 units)
        float l_sum = 0.f;         // running sum of exponentials
        bool ok = true;
        grid_dependency_wait();

        for (int j = 0; j < n_blocks; ++j) {
            const int buf = j & 1;
            const uint32_t buf_phase = static_cast<uint32_t>((j >> 1) & 1);
            if (!mbar_wait_warp(&bar_s_full[buf], buf_phase, abort_word, kDevTimeoutSoftmax)) {
                ok = false;
                break;
            }
            tc_fence_after_sync();
            const uint32_t s_addr = tmem_s0 + lane_base + static_cast<uint32_t>(buf * kChBN);
            const int n_valid = min(kChBN, p.inner - j * kChBN);
            float factor = 1.f;
            if (kSoftmax) {
                float mx = -INFINITY;
#pragma unroll 1
                for (int c = 0; c < kChBN / 32; ++c) {
                    uint32_t r[32];
                    tmem_ld_x32(s_addr + static_cast<uint32_t>(c * 32), r);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        if (c * 32 + i < n_valid) mx = fmaxf(mx, __uint_as_float(r[i]) * p.scale_log2);
                }
                if (j == 0) {
                    m_used = mx;
                } else if (mx > m_used + kRescaleThreshold) {
                    factor = fast_exp2(m_used - mx);
                    m_used = mx;
                }
            }
            // P of the previous block must have been consumed (and O updated) before P / O are touched.
            if (j > 0) {
                if (!mbar_wait_warp(bar_p_empty, static_cast<uint32_t>((j - 1) & 1), abort_word, kDevTimeoutSoftmax)) {
                    ok = false;
                    break;
                }
                tc_fence_after_sync();
            }
            if (kSoftmax) {
                l_sum *= factor;
                if (__any_sync(0xffffffffu, factor != 1.f)) {
#pragma unroll 1
                    for (int c = 0; c < p.dv / 16; ++c) {
                        uint32_t r[16];
                        const uint32_t o_addr = tmem_o + lane_base + static_cast<uint32_t>(c * 16);
                        tmem_ld_x16(o_addr, r);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 16; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * factor);
                        asm volatile(
                            "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
                            "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(o_addr),
                            "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                            "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
                            : "memory");
                    }
                    tmem_st_wait();
                }
            }
            // S -> P (fp16) into swizzled shared memory
#pragma unroll 1
            for (int c = 0; c < kChBN / 32; ++c) {
                uint32_t r[32];
                tmem_ld_x32(s_addr + static_cast<uint32_t>(c * 32), r);
                tmem_ld_wait();
                uint32_t packed[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    float a = __uint_as_float(r[2 * i]);
                    float b = __uint_as_float(r[2 * i + 1]);
                    if (kSoftmax) {
                        a = (c * 32 + 2 * i < n_valid) ? fast_exp2(fmaf(a, p.scale_log2, -m_used)) : 0.f;
                        b = (c * 32 + 2 * i + 1 < n_valid) ? fast_exp2(fmaf(b, p.scale_log2, -m_used)) : 0.f;
                        l_sum += a + b;
                    }
                    packed[i] = pack_half2(a, b);
                }
                // columns [c*32, c*32+32) = 16-byte chunks (c&1)*4 .. +3 of swizzle chunk c>>1
                uint8_t* chunk_base = s_p + (c >> 1) * kChChunk;
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const uint32_t off = sw128_offset(static_cast<uint32_t>(row_in_tile), static_cast<uint32_t>((c & 1) * 4 + q));
                    *reinterpret_cast<uint4*>(chunk_base + off) =
                        make_uint4(packed[4 * q], packed[4 * q + 1], packed[4 * q + 2], packed[4 * q + 3]);
                }
            }
            tc_fence_before_sync();
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&bar_s_empty[buf]);
                mbar_arrive(bar_p_full);
            }
        }

        // ---------------- epilogue ----------------
        if (ok && mbar_wait_warp(bar_o_full, 0, abort_word, kDevTimeoutEpilogue)) {
            tc_fence_after_sync();
            const float inv_l = kSoftmax ? (1.f / l_sum) : 1.f;
            const int64_t out_row = static_cast<int64_t>(bh) * p.rows + row;
            if (!kSoftmax && p.store_by_tma) {
                // fp32 result: 32 x 32 boxes through shared memory (128-byte swizzle) and TMA stores of whole
                // lines. Every MMA has completed, so the operand tile of the second product is free to stage in;
                // TMA clips boxes at the edges of the output.
                uint8_t* stage = s_p + quarter * 8192;
                int sbuf = 0;
                if (lane == 0) tma_prefetch_desc(&tmap_o);
#pragma unroll 1
                for (int c = 0; c < (p.dv + 31) / 32; ++c) {
                    uint32_t r[32];
                    tmem_ld_x32(tmem_o + lane_base + static_cast<uint32_t>(c * 32), r);
                    tmem_ld_wait();
                    if (lane == 0) tma_store_wait_read<1>();
                    __syncwarp();
                    uint8_t* box = stage + sbuf * 4096 + lane * 128;
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        *reinterpret_cast<uint4*>(box + ((j ^ (lane & 7)) << 4)) = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        if (q0 + quarter * 32 < p.rows) tma_store_3d(&tmap_o, stage + sbuf * 4096, c * 32, q0 + quarter * 32, bh);
                        tma_store_commit();
                    }
                    sbuf ^= 1;
                }
                if (lane == 0) tma_store_wait_read<0>();
            } else {
#pragma unroll 1
                for (int c = 0; c < p.dv / 16; ++c) {
                    uint32_t r[16];
                    tmem_ld_x16(tmem_o + lane_base + static_cast<uint32_t>(c * 16), r);
                    tmem_ld_wait();
                    if (row < p.rows) {
                        if (kSoftmax) {
                            uint32_t h[8];
#pragma unroll
                            for (int i = 0; i < 8; ++i)
                                h[i] = pack_half2(__uint_as_float(r[2 * i]) * inv_l, __uint_as_float(r[2 * i + 1]) * inv_l);
                            uint4* dst = reinterpret_cast<uint4*>(static_cast<__half*>(p.out) + out_row * p.dv + c * 16);
                            dst[0] = make_uint4(h[0], h[1], h[2], h[3]);
                            dst[1] = make_uint4(h[4], h[5], h[6], h[7]);
                        } else {
                            float4* dst = reinterpret_cast<float4*>(static_cast<float*>(p.out) + out_row * p.dv + c * 16);
#pragma unroll
                            for (int i = 0; i < 4; ++i)
                                dst[i] = make_float4(__uint_as_float(r[4 * i]), __uint_as_float(r[4 * i + 1]),
                                                     __uint_as_float(r[4 * i + 2]), __uint_as_float(r[4 * i + 3]));
                        }
                    }
                }
            }
            if (kSoftmax && p.lse != nullptr && row < p.rows)
                p.lse[out_row] = (m_used + log2f(l_sum)) * 0.6931471805599453f;
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

// Tensor map over a [batch, rows, cols] fp16 array (cols innermost) with a box of 64 x box_rows x 1.
static int encode_3d(CUtensorMap* out, const void* base, int64_t batch, int64_t rows, int64_t cols, uint32_t box_rows) {
    const uint64_t dims[3] = {static_cast<uint64_t>(cols), static_cast<uint64_t>(rows), static_cast<uint64_t>(batch)};
    const uint64_t strides[2] = {static_cast<uint64_t>(cols) * 2, static_cast<uint64_t>(rows) * static_cast<uint64_t>(cols) * 2};
    const uint32_t box[3] = {64, box_rows, 1};
    return encode_tmap_f16_sw128(out, base, 3, dims, strides, box);
}

template <bool kSoftmax, bool kVTrans>
static int launch_chain(const void* Q, const void* K, const void* V, void* out, float* lse, int64_t batch,
                        int64_t rows, int64_t inner, int64_t dk, int64_t dv, float scale, cudaStream_t stream) {
    const DeviceInfo* dev = nullptr;
    if (int rc = current_device(&dev)) return rc;
    CUtensorMap tq, tk, tv;
    if (int rc = encode_3d(&tq, Q, batch, rows, dk, kChBM)) return rc;
    if (int rc = encode_3d(&tk, K, batch, inner, dk, kChBN)) return rc;
    if (kVTrans) {
        if (int rc = encode_3d(&tv, V, batch, dv, inner, static_cast<uint32_t>(dv))) return rc;
    } else {
        if (int rc = encode_3d(&tv, V, batch, inner, dv, kChBN)) return rc;
    }
    auto kernel = chain_kernel<kSoftmax, kVTrans>;
    static OncePerDevice once;
    if (int rc = raise_smem_limit_once(once, dev->device, kernel, kChSmem)) return rc;
    ChainParams p;
    p.rows = static_cast<int>(rows);
    p.inner = static_cast<int>(inner);
    p.dk = static_cast<int>(dk);
    p.dv = static_cast<int>(dv);
    p.scale_log2 = scale * 1.4426950408889634f;
    p.out = out;
    p.lse = lse;
    p.status = dev->status_word;
    CUtensorMap to;
    memset(&to, 0, sizeof(to));
    p.store_by_tma = 0;
    if (!kSoftmax && aligned16(out) && dv % 4 == 0) {
        if (int rc = encode_tmap_f32_sw128_3d(&to, out, static_cast<uint64_t>(dv), static_cast<uint64_t>(rows),
                                              static_cast<uint64_t>(batch), 32, 32))
            return rc;
        p.store_by_tma = 1;
    }
    const dim3 grid(static_cast<unsigned>((rows + kChBM - 1) / kChBM), static_cast<unsigned>(batch));
    TCB_CUDA(launch_overlapped(kernel, grid, dim3(kChThreads), kChSmem, stream, tq, tk, tv, to, p));
    return TC_OK;
}

static int check_chain_dims(const char* op, int64_t batch, int64_t rows, int64_t inner, int64_t dk, int64_t dv) {
    TCB_REQUIRE(batch > 0 && rows > 0 && inner > 0, "%s: batch, rows and inner extent must be positive", op);
    TCB_REQUIRE(batch <= 65535, "%s: batch (x heads) = %lld exceeds the grid limit 65535", op, (long long)batch);
    TCB_REQUIRE(rows < (1ll << 31) && inner < (1ll << 31), "%s: extent does not fit in 31 bits", op);
    TCB_REQUIRE(dk % 16 == 0 && dk >= 16 && dk <= 128, "%s: first contraction length %lld must be a multiple of 16 in [16,128]",
                op, (long long)dk);
    TCB_REQUIRE(dv % 16 == 0 && dv >= 16 && dv <= 128, "%s: output width %lld must be a multiple of 16 in [16,128]", op,
                (long long)dv);
    return TC_OK;
}

// Two-tile ping-pong attention kernel (attn.cu), used when there is more than one 128-row tile of queries,
// a causal mask or sequence-major operands.
int launch_attn_pingpong(const void* Q, const void* K, const void* V, void* O, float* lse, int64_t batch, int64_t heads,
                         int64_t seq_q, int64_t seq_kv, int64_t dk, int64_t dv, float scale, bool v_trans, bool causal,
                         bool seq_major, cudaStream_t stream);

static int attn_entry(const char* op, const void* Q, const void* K, const void* V, void* O, float* lse, int64_t batch,
                      int64_t heads, int64_t seq_q, int64_t seq_kv, int64_t head_dim, int64_t head_dim_v, float scale,
                      int v_is_transposed, int causal, int seq_major, tc_stream_t stream) {
    TCB_REQUIRE(Q && K && V && O, "%s: null pointer argument", op);
    TCB_REQUIRE(batch > 0 && heads > 0, "%s: batch and heads must be positive", op);
    if (int rc = check_chain_dims(op, batch * heads, seq_q, seq_kv, head_dim, head_dim_v)) return rc;
    TCB_REQUIRE(!v_is_transposed || seq_kv % 8 == 0, "%s: seq_kv = %lld must be a multiple of 8 for transposed V", op,
                (long long)seq_kv);
    TCB_REQUIRE(!(v_is_transposed && seq_major), "%s: a transposed V is not supported with sequence-major operands", op);
    TCB_REQUIRE(head_dim % 8 == 0 && head_dim_v % 8 == 0, "%s: head dims must be multiples of 8", op);
    TCB_REQUIRE(aligned16(Q) && aligned16(K) && aligned16(V) && aligned16(O), "%s: pointers must be 16-byte aligned", op);
    TCB_REQUIRE(isfinite(scale), "%s: scale is not finite", op);
    auto* st = static_cast<cudaStream_t>(stream);
    const bool two_tiles = seq_q > kChBM || causal || seq_major;
    // Both kernels mask after scaling (a masked column is -inf whatever the scale), so scale == 0, which makes every
    // visible KV row weigh the same, needs no special case.
    if (two_tiles)
        return launch_attn_pingpong(Q, K, V, O, lse, batch, heads, seq_q, seq_kv, head_dim, head_dim_v, scale,
                                    v_is_transposed != 0, causal != 0, seq_major != 0, st);
    if (v_is_transposed)
        return launch_chain<true, true>(Q, K, V, O, lse, batch * heads, seq_q, seq_kv, head_dim, head_dim_v, scale, st);
    return launch_chain<true, false>(Q, K, V, O, lse, batch * heads, seq_q, seq_kv, head_dim, head_dim_v, scale, st);
}

}  // namespace tcb

extern "C" int tc_b2b_gemm_f16(const void* A, const void* B, const void* D, void* E, int64_t M, int64_t N, int64_t K,
                               int64_t P, int64_t batch, tc_stream_t stream) {
    using namespace tcb;
    TCB_REQUIRE(A && B && D && E, "b2b_gemm: null pointer argument");
    if (int rc = check_chain_dims("b2b_gemm", batch, M, N, K, P)) return rc;
    TCB_REQUIRE(N % 8 == 0, "b2b_gemm: N = %lld must be a multiple of 8 (rows of D are 16-byte granular)", (long long)N);
    TCB_REQUIRE(aligned16(A) && aligned16(B) && aligned16(D) && aligned16(E), "b2b_gemm: pointers must be 16-byte aligned");
    return launch_chain<false, true>(A, B, D, E, nullptr, batch, M, N, K, P, 1.f, static_cast<cudaStream_t>(stream));
}

extern "C" int tc_flash_attn_fwd_f16(const void* Q, const void* K, const void* V, void* O, float* lse, int64_t batch,
                                     int64_t heads, int64_t seq_q, int64_t seq_kv, int64_t head_dim,
                                     int64_t head_dim_v, float scale, int v_is_transposed, tc_stream_t stream) {
    return tcb::attn_entry("flash_attn_fwd", Q, K, V, O, lse, batch, heads, seq_q, seq_kv, head_dim, head_dim_v, scale,
                           v_is_transposed, 0, 0, stream);
}

extern "C" int tc_flash_attn_fwd_ex_f16(const void* Q, const void* K, const void* V, void* O, float* lse, int64_t batch,
                                        int64_t heads, int64_t seq_q, int64_t seq_kv, int64_t head_dim,
                                        int64_t head_dim_v, float scale, int v_is_transposed, int causal,
                                        int seq_major, tc_stream_t stream) {
    return tcb::attn_entry("flash_attn_fwd_ex", Q, K, V, O, lse, batch, heads, seq_q, seq_kv, head_dim, head_dim_v, scale,
                           v_is_transposed, causal, seq_major, stream);
}
