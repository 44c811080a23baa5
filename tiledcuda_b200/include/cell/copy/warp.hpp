// Which part of a tile a thread touches. The reference derives per-warp sub-tile offsets from the
// WarpLayout grid and the WarpReuse mode (include/cell/copy/warp.hpp:47-204). Here the ownership rule is
// the one tcgen05.ld imposes: with W warps, warp w owns rows [32w, 32w+32) of a 128-row tile (its TMEM
// lane quarter), lane l owns row 32w + l. CTA-wide copies simply stride all threads over 16-byte pieces.
#pragma once

#include "config.hpp"
#include "types/layout.hpp"

namespace tiledcuda::cell::copy::warp {

template <typename WarpLayout_>
struct CopyBase {
    using WarpLayout = WarpLayout_;
    static constexpr int kWarps = static_cast<int>(tl::get_numel<WarpLayout>);
    static constexpr int kThreads = kWarps * 32;

    DEVICE static int warp_id() { return static_cast<int>(threadIdx.x) >> 5; }
    DEVICE static int lane_id() { return static_cast<int>(threadIdx.x) & 31; }
    DEVICE static int warp_row() { return warp_id() / static_cast<int>(tl::num_cols<WarpLayout>); }
    DEVICE static int warp_col() { return warp_id() % static_cast<int>(tl::num_cols<WarpLayout>); }
    // Row of a 128-row tile this thread owns in register fragments (TMEM lane = row).
    DEVICE static int owned_row() { return (warp_id() & 3) * 32 + lane_id(); }
};

}  // namespace tiledcuda::cell::copy::warp
