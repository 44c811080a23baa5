// TmemTile: handle of an fp32 accumulator tile in tensor memory (TMEM).
//
// New on this architecture: the reference accumulates in a register RegTile that every warp owns a piece
// of; tcgen05.mma accumulates into TMEM, 128 lanes (tile rows) by up to 512 32-bit columns per SM. The
// handle is just the TMEM address of the tile's first column; it is what compute::gemm writes and what
// copy::TmemToRegLoader reads. `TmemAllocator` wraps allocation (one warp, power-of-two columns >= 32).
#pragma once

#include <cstdint>

#include "types/layout.hpp"

namespace tiledcuda::cell {

template <typename Element_, typename Layout_>
class TmemTile {
  public:
    using DType = Element_;
    using Layout = Layout_;
    static_assert(sizeof(DType) == 4, "TMEM accumulators are 32-bit");
    static constexpr int kRows = tl::num_rows<Layout>;   // <= 128: rows map to TMEM lanes
    static constexpr int kCols = tl::num_cols<Layout>;   // 32-bit columns
    static_assert(kRows <= traits::Sm100::kMmaM, "an accumulator tile has at most 128 rows");
    static_assert(kCols <= traits::Sm100::kTmemColumns, "an accumulator tile has at most 512 columns");

    HOST_DEVICE TmemTile() : addr_(0) {}
    HOST_DEVICE explicit TmemTile(uint32_t tmem_addr) : addr_(tmem_addr) {}

    // TMEM address (lane in bits 31..16, column in bits 15..0) of column `col`, lane 0.
    HOST_DEVICE uint32_t address(int col = 0) const { return addr_ + static_cast<uint32_t>(col); }

    // Sub-tile of columns [col, col + kSubCols).
    template <int kSubCols>
    HOST_DEVICE TmemTile<DType, tl::RowMajor<kRows, kSubCols>> columns(int col) const {
        return TmemTile<DType, tl::RowMajor<kRows, kSubCols>>(addr_ + static_cast<uint32_t>(col));
    }

  private:
    uint32_t addr_;
};

// Smallest legal TMEM allocation that holds `cols` columns.
HOST_DEVICE constexpr int tmem_alloc_columns(int cols) {
    int c = 32;
    while (c < cols) c *= 2;
    return c;
}

}  // namespace tiledcuda::cell
