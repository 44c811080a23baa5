// LSTM cell: gates = x W^T + h U^T + bias, then the sigmoid / tanh / state update, in one kernel.
//
// A CTA owns 128 batch rows and HT hidden units. Its B operand is gathered from the four gate blocks
// of W (then U): rows [g*H + j0, g*H + j0 + HT) for g = i, f, g, o land next to each other in one
// shared-memory tile, so a single tcgen05.mma with N = 4*HT produces all four gates of those units
// in the same TMEM lanes (= batch rows). The K loop runs over the input features (x against W) and
// continues over the hidden features (h against U) into the same accumulator, so the two gate GEMMs
// are one accumulation chain. The epilogue thread of a batch row reads its i, f, g, o columns,
// applies the nonlinearities in fp32, updates the fp32 cell state and writes h as fp16.
//   warp 0 TMA producer, warp 1 MMA issuer + TMEM owner, warps 2..5 fused epilogue.
//
// The reference snapshot only names this op (Makefile:3 `test_lstm_cell`); the math is that of
// torch.nn.LSTMCell with gate order (i, f, g, o).
#include <mutex>

#include "host.h"
#include "sm100.cuh"

namespace tcb {

// GEMM dispatch for a caller-supplied device record (gemm.cu).
int gemm_f16_f32_on(const DeviceInfo* dev, const void* A, const void* B, float* C, int64_t M, int64_t N, int64_t K,
                    int64_t lda, int64_t ldb, int64_t ldc, cudaStream_t stream, bool bf16, int sm_limit = 0);

constexpr int kLstmBM = 128;
constexpr int kLstmBK = 64;
constexpr int kLstmThreads = 192;

template <int HT>
struct LstmCfg {
    static constexpr int kN = 4 * HT;
    static constexpr int kABytes = kLstmBM * kLstmBK * 2;
    static constexpr int kGateBytes = HT * kLstmBK * 2;
    static constexpr int kBBytes = 4 * kGateBytes;
    // A stage of the ring holds kSub K blocks (each a 64-wide swizzled box per operand) behind ONE barrier: a
    // barrier wait costs either side about 200 cycles even when the phase has completed, against 48 (N = 64) or
    // 64 (N = 128) cycles per MMA, and the tensor pipe runs dry while the issuing thread waits.
    static constexpr int kSub = kN <= 128 ? 2 : 1;
    static constexpr int kBlockBytes = kABytes + kBBytes;
    static constexpr int kStageBytes = kSub * kBlockBytes;
    static constexpr int kStages = (192 * 1024) / kStageBytes;
    static constexpr int kSmem = kStages * kStageBytes + 256 + 1024;
    static constexpr int kTmemCols = kN < 32 ? 32 : kN;
};

struct LstmParams {
    const float* gx;      // [B, 4H] fp32 pre-activations x W^T computed beforehand, or null
    const float* bias;    // [4H] or null
    const float* c_prev;  // [B, H]
    float* c_out;         // [B, H]
    __half* h_out;        // [B, H]
    int batch;
    int input;
    int hidden;
    int zx, zh;           // step index of this launch's x slab and h_prev slab in their [steps, batch, cols] tensor maps
    int early_reads;      // the launch before this one in the stream is a step of the same chain: nothing it writes
                          // (h, c) is read by the prefetch of projections and bias, which may then precede the wait
    uint32_t* status;
};

// The epilogue is bound by the special-function unit (16 results per clock per SM): tanh.approx.f32 is one such
// operation where exp + reciprocal are two, and sigmoid(x) = 0.5 tanh(x / 2) + 0.5 rides on it. Its relative error
// (about 2^-11) is below the fp16 rounding of h; against the fp32 oracle a 64-step chain differs by 2.1e-4
// (relative Frobenius, h) with either formulation.
__device__ __forceinline__ float tanh_f(float x) {
    float y;
    asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float sigmoid_f(float x) { return fmaf(0.5f, tanh_f(0.5f * x), 0.5f); }

template <int HT>
__global__ void __launch_bounds__(kLstmThreads, 1)
lstm_cell_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
                 const __grid_constant__ CUtensorMap tmap_h, const __grid_constant__ CUtensorMap tmap_u,
                 const LstmParams p) {
    using Cfg = LstmCfg<HT>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = align_smem_1024(smem_raw);
    uint8_t* smem_a = smem;
    uint8_t* smem_b = smem + Cfg::kStages * Cfg::kSub * Cfg::kABytes;
    uint64_t* bar_full = reinterpret_cast<uint64_t*>(smem + Cfg::kStages * Cfg::kStageBytes);
    uint64_t* bar_empty = bar_full + Cfg::kStages;
    uint64_t* bar_acc_full = bar_empty + Cfg::kStages;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_acc_full + 1);
    volatile uint32_t* abort_word = tmem_slot + 1;

    // broadcast from lane 0, so that the compiler knows the role of a warp to be the same for all its lanes
    const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0);
    const int lane = threadIdx.x & 31;
    const int j0 = blockIdx.x * HT;        // first hidden unit of this CTA
    const int b0 = blockIdx.y * kLstmBM;   // first batch row
    const int kb_x = p.gx != nullptr ? 0 : (p.input + kLstmBK - 1) / kLstmBK;
    const int kb_h = (p.hidden + kLstmBK - 1) / kLstmBK;
    const int k_blocks = kb_x + kb_h;

    if (threadIdx.x == 0) {
        for (int s = 0; s < Cfg::kStages; ++s) {
            mbar_init(&bar_full[s], 1);
            mbar_init(&bar_empty[s], 1);
        }
        mbar_init(bar_acc_full, 1);
        *abort_word = 0;
        fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, Cfg::kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // The producer and the MMA issuer run as whole warps with one elected lane executing the TMA, MMA and commit
        // instructions: with every lane on the same path the address and descriptor arithmetic stays in the uniform
        // datapath, whose registers those instructions read; behind a branch on the lane index every operand would be
        // moved there first, a fixed cost per instruction that a step of this kernel pays some three hundred times.
        const bool leader = elect_one_sync();
        {
            if (leader) {
                tma_prefetch_desc(&tmap_x);
                tma_prefetch_desc(&tmap_w);
                tma_prefetch_desc(&tmap_h);
                tma_prefetch_desc(&tmap_u);
            }
            int stage = 0;
            uint32_t phase = 0;
            auto load_b = [&](int kbs, int slot, uint64_t* bar) {
                // one 3-D box {64 k, HT units, 4 gates}: the four gate slabs land side by side, gate-major
                const bool from_x = kbs < kb_x;
                const int part = from_x ? kb_x : kb_h;
                const int kcoord = ((from_x ? kbs : kbs - kb_x) + static_cast<int>(blockIdx.x)) % part * kLstmBK;
                tma_load_3d(smem_b + slot * Cfg::kBBytes, from_x ? &tmap_w : &tmap_u, bar, kcoord, j0, 0);
            };
            // h_prev (and c_prev, read by the epilogue) come from the previous launch in the stream: with
            // programmatic dependent launch everything above overlapped its tail, the data is awaited here.
            grid_dependency_wait();
            // Only now may the next step's CTAs start (as SMs free up): they prefetch the hoisted projections before
            // their own wait, which is sound only once everything older than this step, the GEMM that wrote the
            // projections included, has completed. Released before this wait, they could start while that GEMM,
            // which releases its own dependents early, is still running.
            grid_launch_dependents();
            for (int kb = 0; kb < k_blocks; kb += Cfg::kSub) {
                if (!mbar_wait_warp(&bar_empty[stage], phase ^ 1u, abort_word, kDevTimeoutProducer)) break;
                const int subs = min(Cfg::kSub, k_blocks - kb);
                if (leader) mbar_arrive_expect_tx(&bar_full[stage], static_cast<uint32_t>(subs * Cfg::kBlockBytes));
                for (int sub = 0; sub < subs; ++sub) {
                    // Every CTA of a batch tile reads the same x / h tiles: each starts at a different K block
                    // and wraps around, so that at any moment the CTAs pull different lines out of L2.
                    const int kbs = kb + sub;
                    const bool from_x = kbs < kb_x;
                    const int part = from_x ? kb_x : kb_h;
                    const int kcoord = ((from_x ? kbs : kbs - kb_x) + static_cast<int>(blockIdx.x)) % part * kLstmBK;
                    const int slot = stage * Cfg::kSub + sub;
                    if (leader) {
                        tma_load_3d(smem_a + slot * Cfg::kABytes, from_x ? &tmap_x : &tmap_h, &bar_full[stage], kcoord, b0,
                                    from_x ? p.zx : p.zh);
                        load_b(kbs, slot, &bar_full[stage]);
                    }
                }
                if (++stage == Cfg::kStages) {
                    stage = 0;
                    phase ^= 1u;
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        const bool leader = elect_one_sync();
        {
            constexpr uint32_t idesc = make_idesc_f16_f32(kLstmBM, Cfg::kN, false, false);
            // The descriptors of a slot are those of slot 0 plus a constant: no address arithmetic between MMAs,
            // which the pipe would wait for (the issuing thread runs barely one MMA ahead of it).
            const uint64_t a_desc0 = make_smem_desc_sw128(smem_u32(smem_a), 16, 1024);
            const uint64_t b_desc0 = make_smem_desc_sw128(smem_u32(smem_b), 16, 1024);
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int kb = 0; kb < k_blocks; kb += Cfg::kSub) {
                if (!mbar_wait_warp(&bar_full[stage], phase, abort_word, kDevTimeoutMma)) {
                    ok = false;
                    break;
                }
                tc_fence_after_sync();
                const int subs = min(Cfg::kSub, k_blocks - kb);
                for (int sub = 0; sub < subs; ++sub) {
                    const int slot = stage * Cfg::kSub + sub;
                    const uint64_t a_desc = a_desc0 + static_cast<uint64_t>(slot * (Cfg::kABytes >> 4));
                    const uint64_t b_desc = b_desc0 + static_cast<uint64_t>(slot * (Cfg::kBBytes >> 4));
#pragma unroll
                    for (int k = 0; k < kLstmBK / 16; ++k)
                        if (leader)
                            umma_f16_ss(tmem_base, a_desc + static_cast<uint64_t>(k * 2), b_desc + static_cast<uint64_t>(k * 2),
                                        idesc, (kb | sub | k) != 0);
                }
                if (leader) umma_commit(&bar_empty[stage]);
                if (++stage == Cfg::kStages) {
                    stage = 0;
                    phase ^= 1u;
                }
            }
            if (ok && leader) umma_commit(bar_acc_full);
        }
        __syncwarp();
    } else {
        const int quarter = warp & 3;
        const int row = b0 + quarter * 32 + lane;
        // What the first 16 units need besides the accumulator is fetched while the K loop runs: the hoisted input
        // projections and the bias do not depend on the previous step and are read (and summed) before anything is
        // awaited; the old cell state is read as soon as the previous step has finished. Only the nonlinearities
        // and the stores are left behind the last MMA.
        float4 pre[16];
        const bool row_ok = row < p.batch && j0 < p.hidden;
        auto prefetch = [&]() {
#pragma unroll
            for (int i = 0; i < 16; ++i) pre[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (row_ok && p.gx != nullptr) {
                const float* g = p.gx + static_cast<int64_t>(row) * (4 * p.hidden) + j0;
#pragma unroll
                for (int gate = 0; gate < 4; ++gate)
#pragma unroll
                    for (int q = 0; q < 4; ++q) pre[gate * 4 + q] = __ldg(reinterpret_cast<const float4*>(g + gate * p.hidden) + q);
            }
            if (row_ok && p.bias != nullptr) {
#pragma unroll
                for (int gate = 0; gate < 4; ++gate)
#pragma unroll
                    for (int i = 0; i < 16; ++i)
                        reinterpret_cast<float*>(&pre[gate * 4])[i] += __ldg(p.bias + gate * p.hidden + j0 + i);
            }
        };
        // Behind another step of the same chain the prefetch runs before the dependency wait (that step writes
        // neither array); behind anything else (the GEMM that produces the projections, a caller's kernel that
        // may produce the bias) it runs after it, still under the K loop.
        if (p.early_reads != 0) prefetch();
        grid_dependency_wait();
        if (p.early_reads == 0) prefetch();
        float4 c_first[4];
        if (row_ok) {
            const float4* c = reinterpret_cast<const float4*>(p.c_prev + static_cast<int64_t>(row) * p.hidden + j0);
#pragma unroll
            for (int q = 0; q < 4; ++q) c_first[q] = c[q];
        }
        if (mbar_wait_warp(bar_acc_full, 0, abort_word, kDevTimeoutEpilogue)) {
            tc_fence_after_sync();
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
#pragma unroll 1
            for (int u0 = 0; u0 < HT; u0 += 16) {
                uint32_t gi[16], gf[16], gg[16], go[16];
                tmem_ld_x16(taddr + static_cast<uint32_t>(0 * HT + u0), gi);
                tmem_ld_x16(taddr + static_cast<uint32_t>(1 * HT + u0), gf);
                tmem_ld_x16(taddr + static_cast<uint32_t>(2 * HT + u0), gg);
                tmem_ld_x16(taddr + static_cast<uint32_t>(3 * HT + u0), go);
                tmem_ld_wait();
                const int unit0 = j0 + u0;
                if (row < p.batch && unit0 < p.hidden) {
                    // hidden % 16 == 0, so a 16-unit group is either fully inside or fully outside
                    const int64_t off = static_cast<int64_t>(row) * p.hidden + unit0;
                    float c_old[16];
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const float4 v = u0 == 0 ? c_first[q] : *reinterpret_cast<const float4*>(p.c_prev + off + 4 * q);
                        c_old[4 * q] = v.x;
                        c_old[4 * q + 1] = v.y;
                        c_old[4 * q + 2] = v.z;
                        c_old[4 * q + 3] = v.w;
                    }
                    float c_new[16];
                    uint32_t h_new[8];
                    float hv[16];
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        float xi = __uint_as_float(gi[i]);
                        float xf = __uint_as_float(gf[i]);
                        float xg = __uint_as_float(gg[i]);
                        float xo = __uint_as_float(go[i]);
                        if (u0 == 0) {
                            xi += reinterpret_cast<const float*>(&pre[0])[i];
                            xf += reinterpret_cast<const float*>(&pre[4])[i];
                            xg += reinterpret_cast<const float*>(&pre[8])[i];
                            xo += reinterpret_cast<const float*>(&pre[12])[i];
                        } else {
                            if (p.gx != nullptr) {
                                const float* g = p.gx + static_cast<int64_t>(row) * (4 * p.hidden) + unit0 + i;
                                xi += __ldg(g);
                                xf += __ldg(g + p.hidden);
                                xg += __ldg(g + 2 * p.hidden);
                                xo += __ldg(g + 3 * p.hidden);
                            }
                            if (p.bias != nullptr) {
                                xi += __ldg(p.bias + 0 * p.hidden + unit0 + i);
                                xf += __ldg(p.bias + 1 * p.hidden + unit0 + i);
                                xg += __ldg(p.bias + 2 * p.hidden + unit0 + i);
                                xo += __ldg(p.bias + 3 * p.hidden + unit0 + i);
                            }
                        }
                        const float c = sigmoid_f(xf) * c_old[i] + sigmoid_f(xi) * tanh_f(xg);
                        c_new[i] = c;
                        hv[i] = sigmoid_f(xo) * tanh_f(c);
                    }
#pragma unroll
                    for (int i = 0; i < 8; ++i) h_new[i] = pack_half2(hv[2 * i], hv[2 * i + 1]);
#pragma unroll
                    for (int q = 0; q < 4; ++q)
                        *reinterpret_cast<float4*>(p.c_out + off + 4 * q) =
                            make_float4(c_new[4 * q], c_new[4 * q + 1], c_new[4 * q + 2], c_new[4 * q + 3]);
                    uint4* hd = reinterpret_cast<uint4*>(p.h_out + off);
                    hd[0] = make_uint4(h_new[0], h_new[1], h_new[2], h_new[3]);
                    hd[1] = make_uint4(h_new[4], h_new[5], h_new[6], h_new[7]);
                }
            }
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, Cfg::kTmemCols);
    }
    if (threadIdx.x == 0 && *abort_word != 0) atomicMax(p.status, *abort_word);
}

// Activations of all steps, [steps, batch, cols] dense: one map per chain, the step is the third coordinate of a
// load (encoding a map per step costs the host more than the launch itself). Rows past `batch` read as zero.
static int encode_slabs(CUtensorMap* out, const void* base, int64_t steps, int64_t rows, int64_t cols) {
    const uint64_t dims[3] = {static_cast<uint64_t>(cols), static_cast<uint64_t>(rows), static_cast<uint64_t>(steps)};
    const uint64_t strides[2] = {static_cast<uint64_t>(cols) * 2, static_cast<uint64_t>(rows) * static_cast<uint64_t>(cols) * 2};
    const uint32_t box[3] = {kLstmBK, kLstmBM, 1};
    return encode_tmap_f16_sw128(out, base, 3, dims, strides, box);
}

struct LstmWeights {
    CUtensorMap w, u;
    int ht;
};

static int pick_ht(const DeviceInfo* dev, int64_t batch, int64_t hidden) {
    const int64_t ctas16 = ((hidden + 15) / 16) * ((batch + kLstmBM - 1) / kLstmBM);
    return ctas16 <= 2 * dev->sm_count ? 16 : 32;
}

// A [4*hidden, cols] weight matrix seen as [4 gates, hidden, cols]; one box covers 64 columns of HT units of
// all four gates, so a stage's whole B operand is a single TMA operation (TMA is limited by operations
// per second as much as by bytes: four 2 KiB boxes per stage cost more than the 16 KiB A tile).
static int encode_gates(CUtensorMap* out, const void* base, int64_t hidden, int64_t cols, uint32_t ht) {
    const uint64_t dims[3] = {static_cast<uint64_t>(cols), static_cast<uint64_t>(hidden), 4};
    const uint64_t strides[2] = {static_cast<uint64_t>(cols) * 2, static_cast<uint64_t>(hidden) * static_cast<uint64_t>(cols) * 2};
    const uint32_t box[3] = {kLstmBK, ht, 4};
    return encode_tmap_f16_sw128(out, base, 3, dims, strides, box);
}

static int encode_weights(LstmWeights* lw, const DeviceInfo* dev, const void* W, const void* U, int64_t batch,
                          int64_t input, int64_t hidden) {
    lw->ht = pick_ht(dev, batch, hidden);
    if (int rc = encode_gates(&lw->w, W, hidden, input, static_cast<uint32_t>(lw->ht))) return rc;
    return encode_gates(&lw->u, U, hidden, hidden, static_cast<uint32_t>(lw->ht));
}

template <int HT>
static int launch_lstm(const CUtensorMap& tx, const LstmWeights& lw, const CUtensorMap& th, const LstmParams& p,
                       const DeviceInfo* dev, cudaStream_t stream) {
    using Cfg = LstmCfg<HT>;
    auto kernel = lstm_cell_kernel<HT>;
    static OncePerDevice once;
    if (int rc = raise_smem_limit_once(once, dev->device, kernel, Cfg::kSmem)) return rc;
    const dim3 grid(static_cast<unsigned>((p.hidden + HT - 1) / HT), static_cast<unsigned>((p.batch + kLstmBM - 1) / kLstmBM));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(kLstmThreads);
    cfg.dynamicSmemBytes = Cfg::kSmem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    TCB_CUDA(cudaLaunchKernelEx(&cfg, kernel, tx, lw.w, th, lw.u, p));
    return TC_OK;
}

static int lstm_step(const LstmWeights& lw, const float* gx, const float* bias, const CUtensorMap& tx, int64_t zx,
                     const CUtensorMap& th, int64_t zh, const float* c_prev, void* h_out, float* c_out, int64_t batch,
                     int64_t input, int64_t hidden, const DeviceInfo* dev, cudaStream_t stream, bool follows_own_step) {
    LstmParams p;
    p.zx = static_cast<int>(zx);
    p.zh = static_cast<int>(zh);
    p.gx = gx;
    p.bias = bias;
    p.c_prev = c_prev;
    p.c_out = c_out;
    p.h_out = static_cast<__half*>(h_out);
    p.batch = static_cast<int>(batch);
    p.input = static_cast<int>(input);
    p.hidden = static_cast<int>(hidden);
    p.status = dev->status_word;
    p.early_reads = follows_own_step ? 1 : 0;
    return lw.ht == 16 ? launch_lstm<16>(tx, lw, th, p, dev, stream) : launch_lstm<32>(tx, lw, th, p, dev, stream);
}

static int check_lstm(const char* op, const void* W, const void* U, const void* x, const void* h, const float* c,
                      void* h_out, float* c_out, int64_t batch, int64_t input, int64_t hidden) {
    TCB_REQUIRE(W && U && x && h && c && h_out && c_out, "%s: null pointer argument", op);
    TCB_REQUIRE(batch > 0 && input > 0 && hidden > 0, "%s: batch, input and hidden must be positive", op);
    TCB_REQUIRE(input % 8 == 0, "%s: input = %lld must be a multiple of 8", op, (long long)input);
    TCB_REQUIRE(hidden % 16 == 0, "%s: hidden = %lld must be a multiple of 16", op, (long long)hidden);
    TCB_REQUIRE(4 * hidden < (1ll << 31) && batch < (1ll << 31) && input < (1ll << 31), "%s: extent too large", op);
    TCB_REQUIRE(aligned16(W) && aligned16(U) && aligned16(x) && aligned16(h) && aligned16(c) && aligned16(h_out) &&
                    aligned16(c_out),
                "%s: pointers must be 16-byte aligned", op);
    return TC_OK;
}

// The launches of a chain: step t reads x[t] and h[t-1] (h0 for the first) through three tensor maps encoded once.
// gx_all: [steps, batch, 4*hidden] hoisted input projections, or null.
static int lstm_chain_steps(const LstmWeights& lw, const float* gx_all, const float* bias, const void* x, const void* h0,
                            const float* c0, void* h_all, float* c_out, int64_t steps, int64_t batch, int64_t input,
                            int64_t hidden, const DeviceInfo* dev, cudaStream_t st) {
    CUtensorMap tx, th0, th;
    if (int rc = encode_slabs(&tx, x, steps, batch, input)) return rc;
    if (int rc = encode_slabs(&th0, h0, 1, batch, hidden)) return rc;
    if (int rc = encode_slabs(&th, h_all, steps, batch, hidden)) return rc;
    __half* hs = static_cast<__half*>(h_all);
    for (int64_t t = 0; t < steps; ++t) {
        const float* gx = gx_all != nullptr ? gx_all + t * batch * 4 * hidden : nullptr;
        if (int rc = lstm_step(lw, gx, bias, tx, t, t == 0 ? th0 : th, t == 0 ? 0 : t - 1, t == 0 ? c0 : c_out,
                               hs + t * batch * hidden, c_out, batch, input, hidden, dev, st, t > 0))
            return rc;
    }
    return TC_OK;
}

}  // namespace tcb

extern "C" int tc_lstm_cell_f16(const void* W, const void* U, const float* bias, const void* x, const void* h_prev,
                                const float* c_prev, void* h_out, float* c_out, int64_t batch, int64_t input,
                                int64_t hidden, tc_stream_t stream) {
    using namespace tcb;
    if (int rc = check_lstm("lstm_cell", W, U, x, h_prev, c_prev, h_out, c_out, batch, input, hidden)) return rc;
    TCB_REQUIRE(h_out != h_prev, "lstm_cell: h_out must not alias h_prev");
    const DeviceInfo* dev = nullptr;
    if (int rc = current_device(&dev)) return rc;
    LstmWeights lw;
    if (int rc = encode_weights(&lw, dev, W, U, batch, input, hidden)) return rc;
    CUtensorMap tx, th;
    if (int rc = encode_slabs(&tx, x, 1, batch, input)) return rc;
    if (int rc = encode_slabs(&th, h_prev, 1, batch, hidden)) return rc;
    return lstm_step(lw, nullptr, bias, tx, 0, th, 0, c_prev, h_out, c_out, batch, input, hidden, dev,
                     static_cast<cudaStream_t>(stream), false);
}

static int lstm_chain_impl(const void* W, const void* U, const float* bias, const void* x, const void* h0, const float* c0,
                           void* h_all, float* c_out, int64_t steps, int64_t batch, int64_t input, int64_t hidden,
                           float* workspace, cudaStream_t st) {
    using namespace tcb;
    TCB_REQUIRE(steps > 0, "lstm_chain: steps must be positive");
    if (int rc = check_lstm("lstm_chain", W, U, x, h0, c0, h_all, c_out, batch, input, hidden)) return rc;
    TCB_REQUIRE((batch * input) % 8 == 0 && (batch * hidden) % 8 == 0, "lstm_chain: per-step slabs must stay 16-byte aligned");
    const DeviceInfo* dev = nullptr;
    if (int rc = current_device(&dev)) return rc;
    LstmWeights lw;
    if (int rc = encode_weights(&lw, dev, W, U, batch, input, hidden)) return rc;
    if (workspace != nullptr) {
        // The input projections do not depend on the recurrence: x W^T for all steps is one large GEMM
        // ([steps*batch, input] x [input, 4*hidden], fp32 result) and each step adds its slab in the epilogue.
        if (int rc = tc_gemm_f16_f32(x, W, workspace, steps * batch, 4 * hidden, input, input, input, 4 * hidden, st)) return rc;
    }
    return lstm_chain_steps(lw, workspace, bias, x, h0, c0, h_all, c_out, steps, batch, input, hidden, dev, st);
}

extern "C" int tc_lstm_chain_f16(const void* W, const void* U, const float* bias, const void* x, const void* h0,
                                 const float* c0, void* h_all, float* c_out, int64_t steps, int64_t batch,
                                 int64_t input, int64_t hidden, tc_stream_t stream) {
    return lstm_chain_impl(W, U, bias, x, h0, c0, h_all, c_out, steps, batch, input, hidden, nullptr,
                           static_cast<cudaStream_t>(stream));
}

extern "C" int64_t tc_lstm_chain_workspace_bytes(int64_t steps, int64_t batch, int64_t hidden) {
    if (steps <= 0 || batch <= 0 || hidden <= 0) return 0;
    return steps * batch * 4 * hidden * static_cast<int64_t>(sizeof(float));
}

extern "C" int tc_lstm_chain_ws_f16(const void* W, const void* U, const float* bias, const void* x, const void* h0,
                                    const float* c0, void* h_all, float* c_out, int64_t steps, int64_t batch,
                                    int64_t input, int64_t hidden, void* workspace, int64_t workspace_bytes,
                                    tc_stream_t stream) {
    using namespace tcb;
    TCB_REQUIRE(workspace != nullptr, "lstm_chain_ws: workspace is NULL");
    TCB_REQUIRE(workspace_bytes >= tc_lstm_chain_workspace_bytes(steps, batch, hidden),
                "lstm_chain_ws: workspace holds %lld bytes, %lld needed", (long long)workspace_bytes,
                (long long)tc_lstm_chain_workspace_bytes(steps, batch, hidden));
    TCB_REQUIRE(aligned16(workspace), "lstm_chain_ws: workspace must be 16-byte aligned");
    return lstm_chain_impl(W, U, bias, x, h0, c0, h_all, c_out, steps, batch, input, hidden, static_cast<float*>(workspace),
                           static_cast<cudaStream_t>(stream));
}

namespace tcb {

// ---------------------------------------------------------------------------------------------------
// The chain for callers that may not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc at the point where they run the chain: a caller
// inside a stream capture (allocation is illegal there), a real-time or serving loop whose memory
// budget was fixed at start-up, or a plug-in that was handed buffers for inputs and outputs only and has
// no allocator of its own. tc_lstm_chain_ws_f16 asks them for scratch memory they cannot provide, and every
// other entry point may allocate the per-device status word on its first use. This variant needs neither:
// its scratch (the hoisted input projections) and its status word live in the arrays below, which are part
// of the library image. Every GPU that loads the library therefore holds kStaticScratchBytes (+ 16) bytes
// for as long as the library is loaded, whether or not this entry point is ever called.
// ---------------------------------------------------------------------------------------------------
constexpr int64_t kStaticScratchFloats = 16ll * 1024 * 1024;                 // 64 MiB
constexpr int64_t kStaticScratchBytes = kStaticScratchFloats * sizeof(float);
static __device__ __align__(256) float g_static_scratch[kStaticScratchFloats];
static __device__ __align__(256) uint32_t g_static_status[4];

struct StaticDevice {
    bool ready = false;
    DeviceInfo info;          // status_word points at this device's copy of g_static_status
    float* scratch = nullptr;  // this device's copy of g_static_scratch
};
static StaticDevice g_static_dev[64];
static std::mutex g_static_mu;

// Set-up, once per device, with that device current. In host code `g_static_scratch` is only a handle for
// the runtime, not a device address, so the address each device gave its copy is asked for here and that
// is what the kernels receive. Nothing is allocated: cudaGetSymbolAddress and the attribute queries only
// look things up.
static int static_device(const StaticDevice** out) {
    int dev = -1;
    TCB_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(TC_ERR_UNSUPPORTED, "device ordinal %d out of range", dev);
    std::lock_guard<std::mutex> lock(g_static_mu);
    StaticDevice& sd = g_static_dev[dev];
    if (!sd.ready) {
        DeviceInfo d;
        d.device = dev;
        TCB_CUDA(cudaDeviceGetAttribute(&d.cc_major, cudaDevAttrComputeCapabilityMajor, dev));
        TCB_CUDA(cudaDeviceGetAttribute(&d.cc_minor, cudaDevAttrComputeCapabilityMinor, dev));
        TCB_CUDA(cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev));
        TCB_CUDA(cudaDeviceGetAttribute(&d.max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
        if (d.cc_major != 10)
            return fail(TC_ERR_UNSUPPORTED, "device %d is sm_%d%d; these kernels are built for sm_100a only", dev, d.cc_major,
                        d.cc_minor);
        void* scratch = nullptr;
        void* status = nullptr;
        TCB_CUDA(cudaGetSymbolAddress(&scratch, g_static_scratch));
        TCB_CUDA(cudaGetSymbolAddress(&status, g_static_status));
        d.status_word = static_cast<uint32_t*>(status);
        sd.info = d;
        sd.scratch = static_cast<float*>(scratch);
        sd.ready = true;
    }
    *out = &sd;
    return TC_OK;
}

}  // namespace tcb

extern "C" int tc_lstm_chain_static_f16(const void* W, const void* U, const float* bias, const void* x, const void* h0,
                                        const float* c0, void* h_all, float* c_out, int64_t steps, int64_t batch,
                                        int64_t input, int64_t hidden, tc_stream_t stream) {
    using namespace tcb;
    auto* st = static_cast<cudaStream_t>(stream);
    // Argument checks first (they need no device), so that a bad call is refused before anything is set up.
    TCB_REQUIRE(steps >= 0, "lstm_chain_static: steps must not be negative");
    if (steps > 0) {
        if (int rc = check_lstm("lstm_chain_static", W, U, x, h0, c0, h_all, c_out, batch, input, hidden)) return rc;
        TCB_REQUIRE((batch * input) % 8 == 0 && (batch * hidden) % 8 == 0,
                    "lstm_chain_static: per-step slabs must stay 16-byte aligned");
        // The limit is tested by division, so that an absurd `steps` cannot wrap the product past it; within the
        // limit steps * batch (the row count of the hoisted GEMM) is far below 2^31.
        const int64_t bytes_per_step = batch * 4 * hidden * static_cast<int64_t>(sizeof(float));
        if (steps > kStaticScratchBytes / bytes_per_step)
            return fail(TC_ERR_UNSUPPORTED,
                        "lstm_chain_static: %lld steps of %lld bytes of scratch each exceed the %lld bytes built into "
                        "the library; use tc_lstm_chain_ws_f16 with your own workspace or tc_lstm_chain_f16",
                        (long long)steps, (long long)bytes_per_step, (long long)kStaticScratchBytes);
    }
    const StaticDevice* sd = nullptr;
    if (int rc = static_device(&sd)) return rc;
    if (steps == 0) {
        // Status query for this path: its kernels record timeouts in the library's own status word, which
        // tc_device_status() does not see. Synchronises the device; launches nothing.
        uint32_t word = 0;
        TCB_CUDA(cudaDeviceSynchronize());
        TCB_CUDA(cudaMemcpy(&word, sd->info.status_word, sizeof(word), cudaMemcpyDeviceToHost));
        if (word != 0) {
            TCB_CUDA(cudaMemset(sd->info.status_word, 0, 4 * sizeof(uint32_t)));
            return fail(TC_ERR_DEVICE, "lstm_chain_static: a kernel of an earlier call recorded status %u", word);
        }
        return TC_OK;
    }
    const DeviceInfo* dev = &sd->info;
    LstmWeights lw;
    if (int rc = encode_weights(&lw, dev, W, U, batch, input, hidden)) return rc;
    // The GEMM overwrites every float of the scratch region the steps read, so nothing has to be cleared.
    if (int rc = gemm_f16_f32_on(dev, x, W, sd->scratch, steps * batch, 4 * hidden, input, input, input, 4 * hidden, st, false)) return rc;
    return lstm_chain_steps(lw, sd->scratch, bias, x, h0, c0, h_all, c_out, steps, batch, input, hidden, dev, st);
}
