// GEMM on CTA pairs: C[M,N] (fp32) = A[M,K] (fp16) * B (fp16 column-major [K,N] = [N,K] rows), 256x256
// output tiles computed by two CTAs (a cluster of two, one per SM) with tcgen05.mma.cta_group::2.
//
// Each CTA of a pair loads its own 128 rows of A and its own 128 of the 256 B rows per 64-wide K block
// (32 KiB per stage instead of 48 KiB for a lone CTA, so six stages fit and B crosses the L2-to-SM
// fabric once per pair instead of once per CTA). The leader CTA (rank 0) issues the MMAs for both;
// each CTA keeps its 128 accumulator rows in its own TMEM, double-buffered, and runs its own epilogue.
//   warp 0      TMA producer (both CTAs): loads land in the issuing CTA's shared memory and complete on
//               the LEADER's full barrier (no multicast: every byte is fetched by the CTA that uses it);
//   warp 1      TMEM owner (both CTAs); in the leader also the MMA issuer. After each K block it
//               commits to the empty barrier of both CTAs, after each tile to both accumulator-full barriers;
//   warps 2..5  epilogue (both CTAs): tcgen05.ld, fp32 stores, then an arrive on the leader's
//               accumulator-empty barrier (eight arrivals per tile: four warps in each CTA).
// All waits are bounded; the two CTAs meet at a cluster barrier before either frees TMEM or exits.
//
// Stands in for the same reference code as gemm.cu (examples/cpp/01_gemm/02_gemm_all_mem/gemm.hpp:92-155).
#include <stdlib.h>
#include <string.h>

#include "host.h"
#include "sm100.cuh"
#include "epilogue.cuh"

namespace tcb {

constexpr int kPairBM = 128;      // rows per CTA (256 per pair)
constexpr int kPairBN = 256;      // columns per pair tile (128 B rows loaded per CTA)
constexpr int kPairBK = 128;     // two 64-element swizzle chunks per operand and stage
constexpr int kPairStages = 3;
constexpr int kPairThreads = 192;
constexpr int kPairABytes = kPairBM * kPairBK * 2;
constexpr int kPairBBytes = (kPairBN / 2) * kPairBK * 2;
constexpr int kPairStageBytes = kPairABytes + kPairBBytes;
constexpr int kPairStoreBytes = kStoreStageBytes;   // epilogue staging for TMA stores
constexpr int kPairSmem = kPairStages * kPairStageBytes + kPairStoreBytes + 256 + 1024;
constexpr int kPairGroupM = 8;    // pair-tiles (256 rows each) per rasterisation group

__device__ __forceinline__ void pair_tile_coords(int tile, int tiles_m, int tiles_n, int& tm, int& tn) {
    const int per_group = kPairGroupM * tiles_n;
    const int group = tile / per_group;
    const int first_m = group * kPairGroupM;
    const int rows = min(kPairGroupM, tiles_m - first_m);
    const int in_group = tile - group * per_group;
    tm = first_m + in_group % rows;
    tn = in_group / rows;
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kPairThreads, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const __grid_constant__ CUtensorMap tmap_c, float* __restrict__ C, int M, int N, int K, int64_t ldc,
                 int tiles_m, int tiles_n, uint32_t* status, uint32_t idesc_extra, int use_tma_store) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = align_smem_1024(smem_raw);
    uint8_t* smem_a = smem;
    uint8_t* smem_b = smem + kPairStages * kPairABytes;
    uint8_t* smem_store = smem + kPairStages * kPairStageBytes;   // 1024-byte aligned
    uint64_t* bar_full = reinterpret_cast<uint64_t*>(smem_store + kPairStoreBytes);  // used in the leader
    uint64_t* bar_empty = bar_full + kPairStages;      // one per CTA
    uint64_t* bar_acc_full = bar_empty + kPairStages;  // one per CTA
    uint64_t* bar_acc_empty = bar_acc_full + 2;        // used in the leader
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_acc_empty + 2);
    volatile uint32_t* abort_word = tmem_slot + 1;

    // both broadcast from lane 0, so that the compiler knows a warp's role to be the same for all its lanes
    const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0);
    const int lane = threadIdx.x & 31;
    const uint32_t rank = __shfl_sync(0xffffffffu, cluster_ctarank(), 0);   // 0 = leader
    const int pair = blockIdx.x >> 1;
    const int num_pairs = gridDim.x >> 1;
    const int num_tiles = tiles_m * tiles_n;
    const int k_blocks = (K + kPairBK - 1) / kPairBK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kPairStages; ++s) {
            mbar_init(&bar_full[s], 1);
            mbar_init(&bar_empty[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&bar_acc_full[a], 1);
            mbar_init(&bar_acc_empty[a], 8);  // four epilogue warps in each CTA of the pair
        }
        *abort_word = 0;
        fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc_pair(tmem_slot, 512);
        tmem_relinquish_pair();
    }
    tc_fence_before_sync();
    cluster_sync_all();   // barriers of both CTAs are initialised before anyone signals across the pair
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    // No global memory touched so far: a kernel queued behind this one may begin its set-up; this one waits for
    // its predecessor where the producer first loads and where the epilogue first stores.
    grid_launch_dependents();

    if (warp == 0) {
        // ---------------- TMA producer (both CTAs) ----------------
        // The producer runs as a whole warp and one elected lane executes the TMA instructions: with every lane on the
        // same path the address arithmetic stays in the uniform datapath, whose registers those instructions read.
        // The MMA issuer below stays a single lane: its MMAs are long enough (128 cycles each) to hide the operand
        // moves, and the warp-wide form measured slower here (4096^3: 124 against 104 us).
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
            for (int tile = pair; ok && tile < num_tiles; tile += num_pairs) {
                int tm, tn;
                pair_tile_coords(tile, tiles_m, tiles_n, tm, tn);
                const int row_a = tm * (2 * kPairBM) + static_cast<int>(rank) * kPairBM;
                const int row_b = tn * kPairBN + static_cast<int>(rank) * (kPairBN / 2);
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!mbar_wait_warp(&bar_empty[stage], phase ^ 1u, abort_word, kDevTimeoutProducer)) {
                        ok = false;
                        break;
                    }
                    // the leader's full barrier counts the bytes of both CTAs
                    const uint32_t full_addr = map_to_cta(smem_u32(&bar_full[stage]), 0);
                    if (leader) {
                        if (rank == 0) mbar_arrive_expect_tx(&bar_full[stage], 2 * kPairStageBytes);
#pragma unroll
                        for (int c = 0; c < kPairBK / 64; ++c) {
                            tma_load_2d_pair(smem_a + stage * kPairABytes + c * (kPairBM * 128), &tmap_a, full_addr, kb * kPairBK + c * 64, row_a);
                            tma_load_2d_pair(smem_b + stage * kPairBBytes + c * ((kPairBN / 2) * 128), &tmap_b, full_addr, kb * kPairBK + c * 64, row_b);
                        }
                    }
                    if (++stage == kPairStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ---------------- MMA issuer (leader CTA only) ----------------
        if (lane == 0 && rank == 0) {
            const uint32_t idesc = make_idesc_f16_f32(2 * kPairBM, kPairBN, false, false) | idesc_extra;
            const uint32_t desc_hi = smem_desc_hi_sw128(1024);
            const uint32_t a_lo0 = smem_desc_lo(smem_u32(smem_a), 16);
            const uint32_t b_lo0 = smem_desc_lo(smem_u32(smem_b), 16);
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            bool ok = true;
            for (int tile = pair; ok && tile < num_tiles; tile += num_pairs) {
                if (!mbar_wait(&bar_acc_empty[acc], acc_phase ^ 1u, abort_word, kDevTimeoutMma)) break;
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * kPairBN);
                // Two K blocks per round: the second stage's barrier is polled together with the wait for the first,
                // so that sixteen MMAs pay the issuing thread's barrier latency once.
                for (int kb = 0; ok && kb < k_blocks; kb += 2) {
                    const bool two = kb + 1 < k_blocks;
                    const int stage2 = stage + 1 == kPairStages ? 0 : stage + 1;
                    const uint32_t phase2 = stage + 1 == kPairStages ? phase ^ 1u : phase;
                    const bool second_full = two && mbar_try_wait(&bar_full[stage2], phase2);
                    for (int i = 0; i < (two ? 2 : 1); ++i) {
                        if (i == 0 || !second_full) {
                            if (!mbar_wait(&bar_full[stage], phase, abort_word, kDevTimeoutMma)) {
                                ok = false;
                                break;
                            }
                            tc_fence_after_sync();
                        }
                        const uint32_t a_lo = a_lo0 + static_cast<uint32_t>(stage) * (kPairABytes >> 4);
                        const uint32_t b_lo = b_lo0 + static_cast<uint32_t>(stage) * (kPairBBytes >> 4);
#pragma unroll
                        for (int k = 0; k < kPairBK / 16; ++k) {
                            const uint32_t off_a = static_cast<uint32_t>(((k >> 2) * (kPairBM * 128) + (k & 3) * 32) >> 4);
                            const uint32_t off_b = static_cast<uint32_t>(((k >> 2) * ((kPairBN / 2) * 128) + (k & 3) * 32) >> 4);
                            umma_f16_ss_pair(d_tmem, smem_desc_join(a_lo + off_a, desc_hi), smem_desc_join(b_lo + off_b, desc_hi), idesc,
                                             (kb | i | k) != 0);
                        }
                        // the stage is free in both CTAs once these MMAs have read it
                        umma_commit_pair_both(smem_u32(&bar_empty[stage]));
                        if (++stage == kPairStages) {
                            stage = 0;
                            phase ^= 1u;
                        }
                    }
                }
                if (!ok) break;
                umma_commit_pair_both(smem_u32(&bar_acc_full[acc]));
                if (++acc == 2) {
                    acc = 0;
                    acc_phase ^= 1u;
                }
            }
        }
        __syncwarp();
    } else {
        // ---------------- epilogue (both CTAs): TMEM -> registers -> (shared -> TMA store | global) ----------------
        const int quarter = warp & 3;
        int acc = 0;
        uint32_t acc_phase = 0;
        int buf = 0;
        uint8_t* stage = smem_store + quarter * 8192;
        const bool use_tma = use_tma_store != 0;
        if (use_tma && lane == 0) tma_prefetch_desc(&tmap_c);
        grid_dependency_wait();
        for (int tile = pair; tile < num_tiles; tile += num_pairs) {
            int tm, tn;
            pair_tile_coords(tile, tiles_m, tiles_n, tm, tn);
            if (!mbar_wait_warp(&bar_acc_full[acc], acc_phase, abort_word, kDevTimeoutEpilogue)) break;
            tc_fence_after_sync();
            const int row0 = tm * (2 * kPairBM) + static_cast<int>(rank) * kPairBM + quarter * 32;
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(acc * kPairBN);
            store_accumulator_rows<kPairBN>(taddr, C, &tmap_c, stage, buf, row0, tn * kPairBN, M, N, ldc, use_tma, lane);
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&bar_acc_empty[acc]), 0));
            if (++acc == 2) {
                acc = 0;
                acc_phase ^= 1u;
            }
        }
        if (use_tma && lane == 0) tma_store_wait_read<0>();   // shared memory has been read; the grid's completion covers the writes
    }

    // ---------------- teardown: neither CTA frees TMEM or exits while its peer may still touch it ----------------
    tc_fence_before_sync();
    cluster_sync_all();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc_pair(tmem_base, 512);
    }
    if (threadIdx.x == 0 && *abort_word != 0) atomicMax(status, *abort_word);
}

// ---------------------------------------------------------------------------------------------------
// Tall variant: 512x256 output tiles per pair. Each CTA owns 256 rows as two 128-row halves with one
// 256-column accumulator each (all 512 TMEM columns), so a 64-wide K block brings 32 KiB of A and 16 KiB
// of B per CTA for eight MMAs: 48 bytes per MMA clock instead of 64, which is what the lone path from
// L2 into an SM sustains. There is no second accumulator set; instead the two halves are published
// and released separately, so the next tile's MMAs into half 0 start while half 1 is being drained. Both
// halves finish within one K block of each other and an SM writes at about 32 B/clk, so most of the two
// drains (about 4250 cycles each) is exposed: roughly 5 % of a tile at K = 8192, less than the quarter of
// operand traffic this shape saves against 256x256 tiles.
constexpr int kTallBK = 64;
constexpr int kTallStages = 4;
constexpr int kTallRound = 2;   // K blocks issued per barrier round (<= kTallStages)
constexpr int kTallABytes = 2 * kPairBM * kTallBK * 2;          // 256 rows
constexpr int kTallBBytes = (kPairBN / 2) * kTallBK * 2;        // 128 of the 256 B rows
constexpr int kTallStageBytes = kTallABytes + kTallBBytes;
constexpr int kTallSmem = kTallStages * kTallStageBytes + kPairStoreBytes + 256 + 1024;

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kPairThreads, 1)
gemm_pair_tall_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                      const __grid_constant__ CUtensorMap tmap_c, float* __restrict__ C, int M, int N, int K, int64_t ldc,
                      int tiles_m, int tiles_n, uint32_t* status, uint32_t idesc_extra, int use_tma_store) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = align_smem_1024(smem_raw);
    uint8_t* smem_a = smem;
    uint8_t* smem_b = smem + kTallStages * kTallABytes;
    uint8_t* smem_store = smem + kTallStages * kTallStageBytes;   // 1024-byte aligned
    uint64_t* bar_full = reinterpret_cast<uint64_t*>(smem_store + kPairStoreBytes);  // used in the leader
    uint64_t* bar_empty = bar_full + kTallStages;      // one per CTA
    uint64_t* bar_acc_full = bar_empty + kTallStages;  // [half], one per CTA
    uint64_t* bar_acc_empty = bar_acc_full + 2;        // [half], used in the leader
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_acc_empty + 2);
    volatile uint32_t* abort_word = tmem_slot + 1;

    // both broadcast from lane 0, so that the compiler knows a warp's role to be the same for all its lanes
    const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0);
    const int lane = threadIdx.x & 31;
    const uint32_t rank = __shfl_sync(0xffffffffu, cluster_ctarank(), 0);   // 0 = leader
    const int pair = blockIdx.x >> 1;
    const int num_pairs = gridDim.x >> 1;
    const int num_tiles = tiles_m * tiles_n;
    const int k_blocks = (K + kTallBK - 1) / kTallBK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kTallStages; ++s) {
            mbar_init(&bar_full[s], 1);
            mbar_init(&bar_empty[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&bar_acc_full[a], 1);
            mbar_init(&bar_acc_empty[a], 8);  // four epilogue warps in each CTA of the pair
        }
        *abort_word = 0;
        fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc_pair(tmem_slot, 512);
        tmem_relinquish_pair();
    }
    tc_fence_before_sync();
    cluster_sync_all();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    // No global memory touched so far: a kernel queued behind this one may begin its set-up; this one waits for
    // its predecessor where the producer first loads and where the epilogue first stores.
    grid_launch_dependents();

    if (warp == 0) {
        // ---------------- TMA producer (both CTAs) ----------------
        // The producer runs as a whole warp and one elected lane executes the TMA instructions: with every lane on the
        // same path the address arithmetic stays in the uniform datapath, whose registers those instructions read.
        // The MMA issuer below stays a single lane: its MMAs are long enough (128 cycles each) to hide the operand
        // moves, and the warp-wide form measured slower here (4096^3: 124 against 104 us).
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
            for (int tile = pair; ok && tile < num_tiles; tile += num_pairs) {
                int tm, tn;
                pair_tile_coords(tile, tiles_m, tiles_n, tm, tn);
                const int row_a = tm * (4 * kPairBM) + static_cast<int>(rank) * (2 * kPairBM);
                const int row_b = tn * kPairBN + static_cast<int>(rank) * (kPairBN / 2);
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!mbar_wait_warp(&bar_empty[stage], phase ^ 1u, abort_word, kDevTimeoutProducer)) {
                        ok = false;
                        break;
                    }
                    const uint32_t full_addr = map_to_cta(smem_u32(&bar_full[stage]), 0);
                    uint8_t* a_dst = smem_a + stage * kTallABytes;
                    if (leader) {
                        if (rank == 0) mbar_arrive_expect_tx(&bar_full[stage], 2 * kTallStageBytes);
                        tma_load_2d_pair(a_dst, &tmap_a, full_addr, kb * kTallBK, row_a);
                        tma_load_2d_pair(smem_b + stage * kTallBBytes, &tmap_b, full_addr, kb * kTallBK, row_b);
                        tma_load_2d_pair(a_dst + kPairBM * 128, &tmap_a, full_addr, kb * kTallBK, row_a + kPairBM);
                    }
                    if (++stage == kTallStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ---------------- MMA issuer (leader CTA only) ----------------
        if (lane == 0 && rank == 0) {
            const uint32_t idesc = make_idesc_f16_f32(2 * kPairBM, kPairBN, false, false) | idesc_extra;
            const uint32_t desc_hi = smem_desc_hi_sw128(1024);
            const uint32_t a_lo0 = smem_desc_lo(smem_u32(smem_a), 16);
            const uint32_t b_lo0 = smem_desc_lo(smem_u32(smem_b), 16);
            int stage = 0;
            uint32_t phase = 0;
            uint32_t tile_phase = 0;
            bool ok = true;
            // MMAs of one K block: both accumulator halves, then the stage is released in both CTAs.
            auto issue_block = [&](int kb) -> bool {
                const uint32_t a_lo = a_lo0 + static_cast<uint32_t>(stage) * (kTallABytes >> 4);
                const uint32_t b_lo = b_lo0 + static_cast<uint32_t>(stage) * (kTallBBytes >> 4);
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    if (kb == 0) {   // the epilogue of the previous tile has drained this half
                        if (!mbar_wait(&bar_acc_empty[half], tile_phase ^ 1u, abort_word, kDevTimeoutMma)) return false;
                        tc_fence_after_sync();
                    }
                    const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(half * kPairBN);
                    const uint32_t a_half = a_lo + static_cast<uint32_t>(half * ((kPairBM * 128) >> 4));
#pragma unroll
                    for (int k = 0; k < kTallBK / 16; ++k)
                        umma_f16_ss_pair(d_tmem, smem_desc_join(a_half + static_cast<uint32_t>(k * 2), desc_hi),
                                         smem_desc_join(b_lo + static_cast<uint32_t>(k * 2), desc_hi), idesc, (kb | k) != 0);
                    if (kb == k_blocks - 1) {
                        umma_commit_pair_both(smem_u32(&bar_acc_full[half]));
                    }
                }
                umma_commit_pair_both(smem_u32(&bar_empty[stage]));
                if (++stage == kTallStages) {
                    stage = 0;
                    phase ^= 1u;
                }
                return true;
            };
            for (int tile = pair; ok && tile < num_tiles; tile += num_pairs) {
                // kTallRound K blocks per round: the barriers of the later ones are polled together with the wait for
                // the first (their latencies overlap), so that a round of up to 8 * kTallRound MMAs pays the issuing
                // thread's barrier latency once; a block whose poll failed is awaited on its own.
                for (int kb = 0; ok && kb < k_blocks; kb += kTallRound) {
                    bool full[kTallRound] = {};
#pragma unroll
                    for (int i = 1; i < kTallRound; ++i) {
                        const int s2 = stage + i < kTallStages ? stage + i : stage + i - kTallStages;
                        const uint32_t ph2 = stage + i < kTallStages ? phase : phase ^ 1u;
                        full[i] = kb + i < k_blocks && mbar_try_wait(&bar_full[s2], ph2);
                    }
#pragma unroll
                    for (int i = 0; i < kTallRound; ++i) {
                        if (kb + i >= k_blocks) break;
                        if (!full[i]) {
                            if (!mbar_wait(&bar_full[stage], phase, abort_word, kDevTimeoutMma)) {
                                ok = false;
                                break;
                            }
                        }
                        if (i == 0 || !full[i]) tc_fence_after_sync();
                        if (!issue_block(kb + i)) {
                            ok = false;
                            break;
                        }
                    }
                }
                tile_phase ^= 1u;
            }
        }
        __syncwarp();
    } else {
        // ---------------- epilogue (both CTAs), one accumulator half at a time ----------------
        const int quarter = warp & 3;
        uint32_t tile_phase = 0;
        bool ok = true;
        int buf = 0;
        uint8_t* stage = smem_store + quarter * 8192;
        const bool use_tma = use_tma_store != 0;
        if (use_tma && lane == 0) tma_prefetch_desc(&tmap_c);
        grid_dependency_wait();
        for (int tile = pair; ok && tile < num_tiles; tile += num_pairs) {
            int tm, tn;
            pair_tile_coords(tile, tiles_m, tiles_n, tm, tn);
#pragma unroll 1
            for (int half = 0; half < 2; ++half) {
                if (!mbar_wait_warp(&bar_acc_full[half], tile_phase, abort_word, kDevTimeoutEpilogue)) {
                    ok = false;
                    break;
                }
                tc_fence_after_sync();
                const int row0 = tm * (4 * kPairBM) + static_cast<int>(rank) * (2 * kPairBM) + half * kPairBM + quarter * 32;
                const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(half * kPairBN);
                store_accumulator_rows<kPairBN>(taddr, C, &tmap_c, stage, buf, row0, tn * kPairBN, M, N, ldc, use_tma, lane);
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&bar_acc_empty[half]), 0));
            }
            tile_phase ^= 1u;
        }
        if (use_tma && lane == 0) tma_store_wait_read<0>();
    }

    // ---------------- teardown ----------------
    tc_fence_before_sync();
    cluster_sync_all();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc_pair(tmem_base, 512);
    }
    if (threadIdx.x == 0 && *abort_word != 0) atomicMax(status, *abort_word);
}

int launch_gemm_pair_tall(const CUtensorMap& ta, const CUtensorMap& tb, float* C, int M, int N, int K, int64_t ldc,
                          const DeviceInfo* dev, cudaStream_t stream, uint32_t idesc_extra) {
    CUtensorMap tc;
    int use_tma = 0;
    if (int rc = output_store_map(&tc, &use_tma, C, M, N, ldc)) return rc;
    static OncePerDevice once;
    if (int rc = raise_smem_limit_once(once, dev->device, gemm_pair_tall_kernel, kTallSmem)) return rc;
    const int tiles_m = (M + 4 * kPairBM - 1) / (4 * kPairBM);
    const int tiles_n = (N + kPairBN - 1) / kPairBN;
    const int tiles = tiles_m * tiles_n;
    const int max_pairs = dev->sm_count / 2;
    const int pairs = tiles < max_pairs ? tiles : max_pairs;
    TCB_CUDA(launch_overlapped(gemm_pair_tall_kernel, dim3(2 * pairs), dim3(kPairThreads), kTallSmem, stream, ta, tb, tc, C, M, N,
                               K, ldc, tiles_m, tiles_n, dev->status_word, idesc_extra, use_tma));
    return TC_OK;
}

int launch_gemm_pair(const CUtensorMap& ta, const CUtensorMap& tb, float* C, int M, int N, int K, int64_t ldc,
                     const DeviceInfo* dev, cudaStream_t stream, uint32_t idesc_extra) {
    CUtensorMap tc;
    int use_tma = 0;
    if (int rc = output_store_map(&tc, &use_tma, C, M, N, ldc)) return rc;
    static OncePerDevice once;
    if (int rc = raise_smem_limit_once(once, dev->device, gemm_pair_kernel, kPairSmem)) return rc;
    const int tiles_m = (M + 2 * kPairBM - 1) / (2 * kPairBM);
    const int tiles_n = (N + kPairBN - 1) / kPairBN;
    const int tiles = tiles_m * tiles_n;
    const int max_pairs = dev->sm_count / 2;
    const int pairs = tiles < max_pairs ? tiles : max_pairs;
    TCB_CUDA(launch_overlapped(gemm_pair_kernel, dim3(2 * pairs), dim3(kPairThreads), kPairSmem, stream, ta, tb, tc, C, M, N, K,
                               ldc, tiles_m, tiles_n, dev->status_word, idesc_extra, use_tma));
    return TC_OK;
}

}  // namespace tcb
