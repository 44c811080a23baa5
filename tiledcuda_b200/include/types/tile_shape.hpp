// Static shapes: TileShape<d0, d1, ...>, dim_size<i, Shape>, get_numel<Shape>, and the underscore used to
// slice iterators. Counterpart of the reference's include/types/tile_shape.hpp:8-28.
#pragma once

#include <cstddef>

#include "config.hpp"

namespace tiledcuda::cell {

template <int... Dims>
struct TileShape {
    static constexpr int kRank = static_cast<int>(sizeof...(Dims));
    static constexpr int kDims[sizeof...(Dims) > 0 ? sizeof...(Dims) : 1] = {Dims...};
    static constexpr long long kNumel = (1ll * ... * Dims);

    HOST_DEVICE static constexpr int at(int i) { return kDims[i]; }
};

template <int I, typename Shape>
inline constexpr int dim_size = Shape::kDims[I];

template <typename Shape>
inline constexpr long long get_numel = Shape::kNumel;

// `_` selects a whole dimension: iterator(i, _) is row strip i, iterator(_, j) is column strip j.
struct Underscore {};
inline constexpr Underscore _{};

}  // namespace tiledcuda::cell
