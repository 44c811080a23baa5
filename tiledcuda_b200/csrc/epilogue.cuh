// Accumulator epilogue shared by the GEMM kernels: TMEM -> registers -> shared memory -> TMA store.
#pragma once

#include <stdlib.h>
#include <string.h>

#include "host.h"
#include "sm100.cuh"

namespace tcb {

constexpr int kStoreStageBytes = 4 * 2 * 4096;   // per epilogue warp two 32-row x 128-byte boxes

// Tensor map of C for the TMA-store epilogue; *use_tma = 0 (and a zeroed map) when C or its row stride is not
// 16-byte granular, in which case the kernels store from registers.
inline int output_store_map(CUtensorMap* tc, int* use_tma, const float* C, int M, int N, int64_t ldc) {
    memset(tc, 0, sizeof(*tc));
    *use_tma = ((ldc & 3) == 0 && (reinterpret_cast<uintptr_t>(C) & 15u) == 0) ? 1 : 0;
    if (!*use_tma) return TC_OK;
    return encode_tmap_f32_sw128(tc, C, static_cast<uint64_t>(N), static_cast<uint64_t>(M), static_cast<uint64_t>(ldc) * 4, 32, 32);
}

// Drains the 32 rows x kCols columns of an accumulator that one epilogue warp owns (TMEM lanes of its quarter)
// to C. With a tensor map for C the rows go through shared memory in 32 x 32 boxes (128-byte swizzle, the
// layout the map expects) and leave as TMA stores of whole 128-byte lines, which the memory system takes
// far better than 16-byte pieces of 32 different rows per instruction; the bulk-store groups belong to
// lane 0, which also makes sure a staging box has been read out before it is overwritten. TMA clips boxes
// at the edges of C. Without a map (C or ldc not 16-byte granular) each thread stores its own row.
template <int kCols>
__device__ __forceinline__ void store_accumulator_rows(uint32_t taddr, float* __restrict__ C, const CUtensorMap* tmap_c,
                                                       uint8_t* stage, int& buf, int row0, int col0, int M, int N,
                                                       int64_t ldc, bool use_tma, int lane) {
    const int row = row0 + lane;
    float* crow = C + static_cast<int64_t>(row) * ldc;
#pragma unroll 1
    for (int c = 0; c < kCols / 32; ++c) {
        uint32_t r[32];
        tmem_ld_x32(taddr + static_cast<uint32_t>(c * 32), r);
        tmem_ld_wait();
        const int col = col0 + c * 32;
        if (use_tma) {
            if (lane == 0) tma_store_wait_read<1>();   // the box written two chunks ago has left shared memory
            __syncwarp();
            uint8_t* box = stage + buf * 4096 + lane * 128;
#pragma unroll
            for (int j = 0; j < 8; ++j)
                *reinterpret_cast<uint4*>(box + ((j ^ (lane & 7)) << 4)) = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
                if (row0 < M && col < N) tma_store_2d(tmap_c, stage + buf * 4096, col, row0);
                tma_store_commit();
            }
            buf ^= 1;
        } else if (row < M) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
                if (col + j < N) crow[col + j] = __uint_as_float(r[j]);
        }
    }
}

}  // namespace tcb
