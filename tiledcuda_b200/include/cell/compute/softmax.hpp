// Row softmax of a register tile. The reference's version exponentiates without subtracting the row
// maximum and calls itself numerically unstable (include/cell/compute/softmax.hpp:1-5, 27-78); this one
// subtracts the maximum first. One row per thread, so the whole thing is thread-local.
#pragma once

#include "cell/compute/broadcast.hpp"
#include "cell/compute/map.hpp"
#include "cell/compute/reduce.hpp"

namespace tiledcuda::cell::compute {

template <typename Tile, tl::Layout kLayout = tl::Layout::kRowMajor>
struct Softmax {
    using DType = typename Tile::DType;
    using RowValue = RegTile<DType, tl::RowMajor<1, 1>>;

    DEVICE void operator()(const Tile& src, Tile& dst) const {
        static_assert(kLayout == tl::Layout::kRowMajor, "softmax runs along rows");
        RowValue row_max, row_sum;
        MaxReduce<Tile>{}(src, row_max);
#pragma unroll
        for (int i = 0; i < Tile::kNumel; ++i) dst.mutable_data()[i] = src.data()[i];
        BroadcastSub<RowValue, Tile>{}(row_max, dst);
        RegTileExp<Tile>{}(dst, dst);
        SumReduce<Tile>{}(dst, row_sum);
        BroadcastDiv<RowValue, Tile>{}(row_sum, dst);
    }
};

}  // namespace tiledcuda::cell::compute
