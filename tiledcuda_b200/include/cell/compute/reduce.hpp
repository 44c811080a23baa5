// Reductions of register tiles.
//
// In the reference a row of a tile is spread over four lanes of a warp and a reduction ends in shuffles
// (include/cell/compute/reduce.hpp:38, 66-77). With the row-per-thread fragments of tcgen05.ld a ROW
// reduction is a plain loop inside the thread (no shuffle, full fp32), which is what the softmax statistics
// of attention need. A COLUMN reduction runs across the threads of a warp (32 rows) with xor shuffles;
// combining the four warps of a 128-row tile is left to the caller (shared memory).
#pragma once

#include "cell/compute/math_functor.hpp"
#include "cell/warp.hpp"
#include "types/register.hpp"

namespace tiledcuda::cell::compute {

namespace detail {
template <typename Tile, tl::Layout kLayout, typename Functor>
struct Reduce {
    using DType = typename Tile::DType;

    // Row-wise: dst(0, 0) = reduce_j src(0, j)
    template <typename DstTile>
    DEVICE void operator()(const Tile& src, DstTile& dst) const {
        static_assert(Tile::kRows == 1, "fragments hold one row per thread");
        Functor f;
        if constexpr (kLayout == tl::Layout::kRowMajor) {
            static_assert(DstTile::kNumel == 1, "a row reduction yields one value per thread");
            // four independent partial results keep the dependency chains short
            DType p0 = src(0, 0), p1 = src(0, Tile::kCols > 1 ? 1 : 0), p2 = src(0, Tile::kCols > 2 ? 2 : 0),
                  p3 = src(0, Tile::kCols > 3 ? 3 : 0);
            if constexpr (Tile::kCols >= 8 && Tile::kCols % 4 == 0) {
#pragma unroll
                for (int j = 4; j < Tile::kCols; j += 4) {
                    p0 = f(p0, src(0, j));
                    p1 = f(p1, src(0, j + 1));
                    p2 = f(p2, src(0, j + 2));
                    p3 = f(p3, src(0, j + 3));
                }
                dst(0, 0) = f(f(p0, p1), f(p2, p3));
            } else {
                DType acc = src(0, 0);
#pragma unroll
                for (int j = 1; j < Tile::kCols; ++j) acc = f(acc, src(0, j));
                dst(0, 0) = acc;
            }
        } else {
            // Column-wise over the 32 rows a warp owns: every lane ends with the reduced value of each column.
            static_assert(DstTile::kNumel == Tile::kCols, "a column reduction yields one value per column");
#pragma unroll
            for (int j = 0; j < Tile::kCols; ++j) {
                DType v = src(0, j);
#pragma unroll
                for (int m = 16; m > 0; m >>= 1) v = f(v, shuffle_xor_sync(v, m));
                dst.mutable_data()[j] = v;
            }
        }
    }
};
}  // namespace detail

template <typename Tile, tl::Layout kLayout = tl::Layout::kRowMajor>
using SumReduce = detail::Reduce<Tile, kLayout, Add<typename Tile::DType>>;

template <typename Tile, tl::Layout kLayout = tl::Layout::kRowMajor>
using MaxReduce = detail::Reduce<Tile, kLayout, Max<typename Tile::DType>>;

}  // namespace tiledcuda::cell::compute
