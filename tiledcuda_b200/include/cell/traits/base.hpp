// Hardware constants the tile types are built around. The reference fixes a 16x16 BaseTile (the mma.sync
// m16n8k16 footprint) and 128-bit accesses (include/cell/traits/base.hpp:16-39). On sm_100a the fixed
// quantities are the tcgen05.mma shape (M = 128 rows per CTA, K = 16 for 16-bit inputs), the 128-byte
// swizzle row (64 fp16) with its 8-row atom, and the 32-lane TMEM quarter a warp can read. BaseTileShape
// keeps its name and its 16x16 value, because tile extents are still counted in multiples of 16.
#pragma once

#include <type_traits>

#if defined(__CUDACC__)
#include <cuda_fp16.h>
#endif

namespace tiledcuda::cell::traits {

#if defined(__CUDACC__)
template <typename T>
inline constexpr bool is_base_type = std::is_same_v<T, float> || std::is_same_v<T, __half>;
#else
template <typename T>
inline constexpr bool is_base_type = std::is_same_v<T, float> || sizeof(T) == 2;
#endif

template <typename Element>
struct BaseTileShape {
    static constexpr int kTileSize = 16;
    static constexpr int kRows = kTileSize;
    static constexpr int kCols = kTileSize;
    static constexpr int kNumel = kRows * kCols;
};

template <typename Element>
struct TraitsBase {
    static constexpr int kAccessInBits = 128;                                 // widest per-thread access
    static constexpr int kElmentBits = static_cast<int>(sizeof(Element)) * 8;
    static constexpr int kNumPerAccess = kAccessInBits / kElmentBits;
};

// tcgen05 / TMA constants
struct Sm100 {
    static constexpr int kMmaM = 128;          // accumulator rows of one CTA (TMEM lanes)
    static constexpr int kMmaK = 16;           // K per tcgen05.mma for 16-bit inputs
    static constexpr int kMaxMmaN = 256;       // widest accumulator of one instruction
    static constexpr int kSwizzleBytes = 128;  // one swizzled shared-memory row
    static constexpr int kSwizzleRows = 8;     // rows per swizzle atom (1024 bytes)
    static constexpr int kTmemColumns = 512;   // 32-bit columns per lane
    static constexpr int kLanesPerWarp = 32;   // TMEM lanes a warp may touch: 32 * (warp % 4) ...
};

}  // namespace tiledcuda::cell::traits
