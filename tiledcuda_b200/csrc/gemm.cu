// GEMM  C[M,N] (fp32) = A[M,K] (fp16, row-major) * B (fp16, column-major [K,N] = [N,K] row-major).
//
// Persistent, warp-specialised sm_100a kernel, one CTA per SM:
//   warp 0      TMA producer: 128x64 A tiles and BNx64 B tiles, 128-byte swizzle, into a ring of
//               shared-memory stages guarded by full/empty mbarriers;
//   warp 1      allocates TMEM and issues tcgen05.mma (M=128, N=BN, K=16; fp16 in, fp32 accumulate),
//               tcgen05.commit releases each stage and publishes each finished accumulator;
//   warps 2..5  epilogue: tcgen05.ld the accumulator (one row per thread) and store fp32 rows.
// Two accumulators live in TMEM (2 x BN columns), so the epilogue of tile i overlaps the main loop
// of tile i+1. Tiles are walked in groups of kGroupM row-tiles so that the CTAs in flight share A and
// B tiles through L2. Loads outside the matrices are zero-filled by TMA; stores are predicated.
//
// Stands in for the reference's `gemm` (examples/cpp/01_gemm/02_gemm_all_mem/gemm.hpp:92-155: cp.async
// -> swizzled smem -> ldmatrix -> mma.sync, single stage) and cell::compute::gemm
// (include/cell/compute/gemm.hpp:19-88).
#include <stdint.h>
#include <stdlib.h>

#include "host.h"
#include "sm100.cuh"
#include "epilogue.cuh"

namespace tcb {

constexpr int kGemmBM = 128;
constexpr int kGemmBK = 64;
constexpr int kGemmThreads = 192;
constexpr int kGroupM = 16;

template <int BN, int STAGES>
struct GemmSmem {
    static constexpr int kABytes = kGemmBM * kGemmBK * 2;
    static constexpr int kBBytes = BN * kGemmBK * 2;
    static constexpr int kStageBytes = kABytes + kBBytes;
    // STAGES counts K blocks of capacity. With BN = 128 a K block is four 64-cycle MMAs, less than the ~200 cycles
    // a barrier wait costs the producer or the issuing thread even on a completed phase, so two K blocks share
    // one ring stage and one barrier; with BN = 256 a K block is 512 cycles of MMA and the wait hides behind it.
    static constexpr int kSub = (BN <= 128 && STAGES % 2 == 0) ? 2 : 1;
    static constexpr int kRing = STAGES / kSub;
    static constexpr int kBarBytes = 256;
    static constexpr int kTotal = STAGES * kStageBytes + kStoreStageBytes + kBarBytes + 1024;  // + slack for 1024-B alignment
};

__device__ __forceinline__ void gemm_tile_coords(int tile, int tiles_m, int tiles_n, int& tm, int& tn) {
    const int per_group = kGroupM * tiles_n;
    const int group = tile / per_group;
    const int first_m = group * kGroupM;
    const int rows = min(kGroupM, tiles_m - first_m);
    const int in_group = tile - group * per_group;
    tm = first_m + in_group % rows;
    tn = in_group / rows;
}

template <int BN, int STAGES>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_f16_f32_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                    const __grid_constant__ CUtensorMap tmap_c, float* __restrict__ C, int M, int N, int K, int64_t ldc,
                    int tiles_m, int tiles_n, uint32_t* status, uint32_t idesc_extra, int use_tma_store) {
    using S = GemmSmem<BN, STAGES>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = align_smem_1024(smem_raw);
    uint8_t* smem_a = smem;
    uint8_t* smem_b = smem + STAGES * S::kABytes;
    uint8_t* smem_store = smem + STAGES * S::kStageBytes;   // 1024-byte aligned
    uint64_t* bar_full = reinterpret_cast<uint64_t*>(smem_store + kStoreStageBytes);
    uint64_t* bar_empty = bar_full + STAGES;
    uint64_t* bar_acc_full = bar_empty + STAGES;
    uint64_t* bar_acc_empty = bar_acc_full + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_acc_empty + 2);
    volatile uint32_t* abort_word = tmem_slot + 1;

    // broadcast from lane 0, so that the compiler knows the role of a warp to be the same for all its lanes
    const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0);
    const int lane = threadIdx.x & 31;
    const int num_tiles = tiles_m * tiles_n;
    const int k_blocks = (K + kGemmBK - 1) / kGemmBK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&bar_full[s], 1);
            mbar_init(&bar_empty[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&bar_acc_full[a], 1);
            mbar_init(&bar_acc_empty[a], 4);  // one arrival per epilogue warp
        }
        *abort_word = 0;
        fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, 2 * BN);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    // Everything above touched no global memory. A kernel queued behind this one may now start its own set-up
    // on SMs this grid leaves free; this kernel in turn waits for the one before it only where it first reads
    // (the producer) or writes (the epilogue) global memory.
    grid_launch_dependents();

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        // Producer and MMA issuer run as whole warps; one elected lane executes the TMA, MMA and commit instructions.
        // With every lane on the same path the address and descriptor arithmetic stays in the uniform datapath, whose
        // registers those instructions read; behind a branch on the lane index every operand is moved there first.
        const bool leader = elect_one_sync();
        {
            if (leader) {
                tma_prefetch_desc(&tmap_a);
                tma_prefetch_desc(&tmap_b);
            }
            grid_dependency_wait();
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
                int tm, tn;
                gemm_tile_coords(tile, tiles_m, tiles_n, tm, tn);
                for (int kb = 0; kb < k_blocks; kb += S::kSub) {
                    if (!mbar_wait_warp(&bar_empty[stage], phase ^ 1u, abort_word, kDevTimeoutProducer)) {
                        ok = false;
                        break;
                    }
                    const int subs = min(S::kSub, k_blocks - kb);
                    if (leader) {
                        mbar_arrive_expect_tx(&bar_full[stage], static_cast<uint32_t>(subs * S::kStageBytes));
                        for (int sub = 0; sub < subs; ++sub) {
                            const int slot = stage * S::kSub + sub;
                            tma_load_2d(smem_a + slot * S::kABytes, &tmap_a, &bar_full[stage], (kb + sub) * kGemmBK, tm * kGemmBM);
                            tma_load_2d(smem_b + slot * S::kBBytes, &tmap_b, &bar_full[stage], (kb + sub) * kGemmBK, tn * BN);
                        }
                    }
                    if (++stage == S::kRing) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        const bool leader = elect_one_sync();
        {
            const uint32_t idesc = make_idesc_f16_f32(kGemmBM, BN, false, false) | idesc_extra;
            const uint64_t a_desc0 = make_smem_desc_sw128(smem_u32(smem_a), 16, 1024);
            const uint64_t b_desc0 = make_smem_desc_sw128(smem_u32(smem_b), 16, 1024);
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
                if (!mbar_wait_warp(&bar_acc_empty[acc], acc_phase ^ 1u, abort_word, kDevTimeoutMma)) break;
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BN);
                for (int kb = 0; kb < k_blocks; kb += S::kSub) {
                    if (!mbar_wait_warp(&bar_full[stage], phase, abort_word, kDevTimeoutMma)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    const int subs = min(S::kSub, k_blocks - kb);
                    for (int sub = 0; sub < subs; ++sub) {
                        // the descriptor of a slot is that of slot 0 plus a constant (address field in 16-byte units)
                        const int slot = stage * S::kSub + sub;
                        const uint64_t a_desc = a_desc0 + static_cast<uint64_t>(slot * (S::kABytes >> 4));
                        const uint64_t b_desc = b_desc0 + static_cast<uint64_t>(slot * (S::kBBytes >> 4));
#pragma unroll
                        for (int k = 0; k < kGemmBK / 16; ++k) {
                            // +32 bytes per K=16 step inside the 128-byte swizzle row
                            if (leader)
                                umma_f16_ss(d_tmem, a_desc + static_cast<uint64_t>(k * 2), b_desc + static_cast<uint64_t>(k * 2),
                                            idesc, (kb | sub | k) != 0);
                        }
                    }
                    if (leader) umma_commit(&bar_empty[stage]);
                    if (++stage == S::kRing) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (!ok) break;
                if (leader) umma_commit(&bar_acc_full[acc]);
                if (++acc == 2) {
                    acc = 0;
                    acc_phase ^= 1u;
                }
            }
        }
        __syncwarp();
    } else {
        // ---------------- epilogue: TMEM -> registers -> (shared -> TMA store | global) ----------------
        const int quarter = warp & 3;  // TMEM lane quarter this warp may read
        int acc = 0;
        uint32_t acc_phase = 0;
        int buf = 0;
        uint8_t* stage = smem_store + quarter * 8192;
        const bool use_tma = use_tma_store != 0;
        if (use_tma && lane == 0) tma_prefetch_desc(&tmap_c);
        grid_dependency_wait();
        for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
            int tm, tn;
            gemm_tile_coords(tile, tiles_m, tiles_n, tm, tn);
            if (!mbar_wait_warp(&bar_acc_full[acc], acc_phase, abort_word, kDevTimeoutEpilogue)) break;
            tc_fence_after_sync();
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(acc * BN);
            store_accumulator_rows<BN>(taddr, C, &tmap_c, stage, buf, tm * kGemmBM + quarter * 32, tn * BN, M, N, ldc, use_tma, lane);
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bar_acc_empty[acc]);
            if (++acc == 2) {
                acc = 0;
                acc_phase ^= 1u;
            }
        }
        if (use_tma && lane == 0) tma_store_wait_read<0>();   // shared memory has been read; the grid's completion covers the writes
    }

    // ---------------- teardown ----------------
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, 2 * BN);
    }
    if (threadIdx.x == 0 && *abort_word != 0) atomicMax(status, *abort_word);
}

template <int BN, int STAGES>
static int launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, float* C, int M, int N, int K, int64_t ldc,
                       const DeviceInfo* dev, cudaStream_t stream, uint32_t idesc_extra) {
    using S = GemmSmem<BN, STAGES>;
    auto kernel = gemm_f16_f32_kernel<BN, STAGES>;
    static OncePerDevice once;
    if (int rc = raise_smem_limit_once(once, dev->device, kernel, S::kTotal)) return rc;
    const int tiles_m = (M + kGemmBM - 1) / kGemmBM;
    const int tiles_n = (N + BN - 1) / BN;
    const int tiles = tiles_m * tiles_n;
    const int grid = tiles < dev->sm_count ? tiles : dev->sm_count;
    CUtensorMap tc;
    int use_tma = 0;
    if (int rc = output_store_map(&tc, &use_tma, C, M, N, ldc)) return rc;
    TCB_CUDA(launch_overlapped(kernel, dim3(grid), dim3(kGemmThreads), S::kTotal, stream, ta, tb, tc, C, M, N, K, ldc, tiles_m,
                               tiles_n, dev->status_word, idesc_extra, use_tma));
    return TC_OK;
}

// 256x256 tiles on CTA pairs (gemm_pair.cu); tb must have been encoded with a 64 x 128 box.
int launch_gemm_pair(const CUtensorMap& ta, const CUtensorMap& tb, float* C, int M, int N, int K, int64_t ldc,
                     const DeviceInfo* dev, cudaStream_t stream, uint32_t idesc_extra);

// 512x256 tiles on CTA pairs (gemm_pair.cu); same tensor maps as launch_gemm_pair.
int launch_gemm_pair_tall(const CUtensorMap& ta, const CUtensorMap& tb, float* C, int M, int N, int K, int64_t ldc,
                          const DeviceInfo* dev, cudaStream_t stream, uint32_t idesc_extra);

// Tile shape for a problem on a device with sm_count SMs: TC_GEMM_TILE_* of the public header.
// A small cost model: waves over the machine times the tensor-pipe cycles one K step of 16 costs in that tile
// (measured: 128 for a 256x256 pair tile; about 160 for a lone 128x256 tile and 128 for a lone 128x128 tile, both
// held back by shared-memory bandwidth, which the TMA writes and the MMA operand reads share), plus the exposed
// epilogue of the last wave. Long K loops over many tiles take 512x256 pair tiles, which fetch a quarter fewer
// operand bytes per FLOP and expose only about one percent of a tile's epilogue (measured: 8192^3 1484 against
// 1456 TFLOP/s, 16384^3 1446 against 1262; equal at 4096^3 and 6144^3; with K = 2048 the square tiles win, 1326
// against 1284).
int gemm_tile_plan(int64_t M, int64_t N, int64_t K, int sm_count) {
    const int64_t k16 = (K + 15) / 16;
    const int64_t pairs = sm_count / 2;
    const int64_t tiles_pair = ((M + 255) / 256) * ((N + 255) / 256);
    const int64_t tiles256 = ((M + 127) / 128) * ((N + 255) / 256);
    const int64_t tiles128 = ((M + 127) / 128) * ((N + 127) / 128);
    const int64_t cost_pair = pairs > 0 ? ((tiles_pair + pairs - 1) / pairs) * (128 * k16) + 1500 : INT64_MAX;
    const int64_t cost_256 = ((tiles256 + sm_count - 1) / sm_count) * (160 * k16) + 1500;
    const int64_t cost_128 = ((tiles128 + sm_count - 1) / sm_count) * (128 * k16) + 800;
    if (N > 128 && M > 128 && cost_pair <= cost_256 && cost_pair <= cost_128) {
        const int64_t tiles_tall = ((M + 511) / 512) * ((N + 255) / 256);
        return (K >= 4096 && tiles_tall >= 4 * pairs) ? TC_GEMM_TILE_PAIR_512x256 : TC_GEMM_TILE_PAIR_256x256;
    }
    if (N > 128 && cost_128 > cost_256) return TC_GEMM_TILE_128x256;
    // A single partial wave of 128x128 tiles: halving the tile width doubles the busy SMs, and although an N = 64
    // MMA runs at two thirds of the rate (shared-memory bound) each CTA's K loop and epilogue get shorter.
    const int64_t tiles64 = ((M + 127) / 128) * ((N + 63) / 64);
    if (N <= 64 || (2 * tiles128 <= sm_count && tiles64 <= sm_count)) return TC_GEMM_TILE_128x64;
    return TC_GEMM_TILE_128x128;
}

// The dispatch of tc_gemm_f16_f32 for a caller that brings its own device record (and therefore its own
// status word) instead of the lazily allocated per-device one. Arguments are trusted: the caller has
// validated them. Used by entry points that must not allocate.
int gemm_f16_f32_on(const DeviceInfo* dev_full, const void* A, const void* B, float* C, int64_t M, int64_t N, int64_t K,
                    int64_t lda, int64_t ldb, int64_t ldc, cudaStream_t stream, bool bf16, int sm_limit) {
    // With an SM budget the tile plan and the persistent grids are sized for that many SMs, the rest stay free
    // for whatever else the caller runs beside the GEMM (a collective that assembles finished blocks, say).
    DeviceInfo limited = *dev_full;
    if (sm_limit > 0 && sm_limit < limited.sm_count) limited.sm_count = sm_limit;
    const DeviceInfo* dev = &limited;
    const uint32_t extra = bf16 ? kIdescBf16Inputs : 0u;
    const int plan = gemm_tile_plan(M, N, K, dev->sm_count);
    const bool use_pair = plan == TC_GEMM_TILE_PAIR_256x256 || plan == TC_GEMM_TILE_PAIR_512x256;
    const uint32_t bn = plan == TC_GEMM_TILE_128x256 ? 256u : (plan == TC_GEMM_TILE_128x64 ? 64u : 128u);
    CUtensorMap ta, tb;
    {
        const uint64_t dims[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(M)};
        const uint64_t strides[1] = {static_cast<uint64_t>(lda) * 2};
        const uint32_t box[2] = {kGemmBK, kGemmBM};
        if (int rc = encode_tmap_f16_sw128(&ta, A, 2, dims, strides, box, bf16)) return rc;
    }
    {
        const uint64_t dims[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(N)};
        const uint64_t strides[1] = {static_cast<uint64_t>(ldb) * 2};
        const uint32_t box[2] = {kGemmBK, bn};
        if (int rc = encode_tmap_f16_sw128(&tb, B, 2, dims, strides, box, bf16)) return rc;
    }
    if (plan == TC_GEMM_TILE_PAIR_512x256) return launch_gemm_pair_tall(ta, tb, C, (int)M, (int)N, (int)K, ldc, dev, stream, extra);
    if (use_pair) return launch_gemm_pair(ta, tb, C, (int)M, (int)N, (int)K, ldc, dev, stream, extra);
    if (plan == TC_GEMM_TILE_128x64) return launch_gemm<64, 8>(ta, tb, C, (int)M, (int)N, (int)K, ldc, dev, stream, extra);
    if (plan == TC_GEMM_TILE_128x128) return launch_gemm<128, 6>(ta, tb, C, (int)M, (int)N, (int)K, ldc, dev, stream, extra);
    return launch_gemm<256, 4>(ta, tb, C, (int)M, (int)N, (int)K, ldc, dev, stream, extra);
}

}  // namespace tcb

static int gemm_entry(const char* op, bool bf16, const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K,
                      int64_t lda, int64_t ldb, int64_t ldc, tc_stream_t stream, int sm_limit = 0) {
    using namespace tcb;
    TCB_REQUIRE(A && B && C, "%s: null pointer argument", op);
    TCB_REQUIRE(M > 0 && N > 0 && K > 0, "%s: M, N, K must be positive (got %lld, %lld, %lld)", op, (long long)M,
                (long long)N, (long long)K);
    TCB_REQUIRE(M < (1ll << 31) && N < (1ll << 31) && K < (1ll << 31), "%s: a dimension does not fit in 31 bits", op);
    TCB_REQUIRE(K % 8 == 0, "%s: K = %lld is not a multiple of 8 (TMA rows are 16-byte granular)", op, (long long)K);
    TCB_REQUIRE(lda >= K && ldb >= K && ldc >= N, "%s: leading dimension smaller than the row length", op);
    TCB_REQUIRE(lda % 8 == 0 && ldb % 8 == 0, "%s: lda and ldb must be multiples of 8 elements (16 bytes)", op);
    TCB_REQUIRE(aligned16(A) && aligned16(B), "%s: A and B must be 16-byte aligned", op);
    TCB_REQUIRE((reinterpret_cast<uintptr_t>(C) & 3u) == 0, "%s: C must be 4-byte aligned", op);
    const DeviceInfo* dev = nullptr;
    if (int rc = current_device(&dev)) return rc;
    // Large problems run 256x256 tiles on CTA pairs; narrow or small ones take lone CTAs with 128x256 or
    // 128x128 tiles so that more SMs are busy (the choice is made in gemm_f16_f32_on).
    return gemm_f16_f32_on(dev, A, B, static_cast<float*>(C), M, N, K, lda, ldb, ldc, static_cast<cudaStream_t>(stream), bf16,
                           sm_limit);
}

extern "C" int tc_gemm_f16_f32(const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K, int64_t lda,
                               int64_t ldb, int64_t ldc, tc_stream_t stream) {
    return gemm_entry("gemm", false, A, B, C, M, N, K, lda, ldb, ldc, stream);
}

extern "C" int tc_gemm_f16_f32_sms(const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K, int64_t lda,
                                   int64_t ldb, int64_t ldc, int max_sms, tc_stream_t stream) {
    using namespace tcb;
    TCB_REQUIRE(max_sms >= 0, "gemm_sms: max_sms must not be negative (0 = all SMs)");
    TCB_REQUIRE(max_sms == 0 || max_sms >= 2, "gemm_sms: a budget needs at least 2 SMs (one CTA pair)");
    return gemm_entry("gemm_sms", false, A, B, C, M, N, K, lda, ldb, ldc, stream, max_sms);
}

extern "C" int tc_gemm_bf16_f32(const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K, int64_t lda,
                                int64_t ldb, int64_t ldc, tc_stream_t stream) {
    return gemm_entry("gemm_bf16", true, A, B, C, M, N, K, lda, ldb, ldc, stream);
}

extern "C" int tc_gemm_tile_plan(int64_t M, int64_t N, int64_t K, int sm_count) {
    using namespace tcb;
    TCB_REQUIRE(M > 0 && N > 0 && K > 0 && sm_count > 0, "gemm_tile_plan: M, N, K and sm_count must be positive");
    return gemm_tile_plan(M, N, K, sm_count);
}
