// Element-wise maps over register tiles (reference: include/cell/compute/map.hpp:17-133). Nested tiles
// are walked recursively; unary maps may change the element type (RegTileConvert).
#pragma once

#include "cell/compute/math_functor.hpp"
#include "types/register.hpp"

namespace tiledcuda::cell::compute {

namespace detail {
template <typename Tile, typename Functor>
struct ElementWise {
    using DType = typename Tile::DType;
    DEVICE void operator()(const Tile& src, Tile& dst) const {
        Functor f;
#pragma unroll
        for (int i = 0; i < Tile::kNumel; ++i) {
            if constexpr (cell::detail::is_reg_tile<DType>::value)
                ElementWise<DType, Functor>{}(src.data()[i], dst.mutable_data()[i]);
            else
                f(src.data()[i], dst.mutable_data()[i]);
        }
    }
};
template <typename Tile, typename Functor>
struct ElementWise2 {
    using DType = typename Tile::DType;
    DEVICE void operator()(const Tile& a, const Tile& b, Tile& dst) const {
        Functor f;
#pragma unroll
        for (int i = 0; i < Tile::kNumel; ++i) {
            if constexpr (cell::detail::is_reg_tile<DType>::value)
                ElementWise2<DType, Functor>{}(a.data()[i], b.data()[i], dst.mutable_data()[i]);
            else
                f(a.data()[i], b.data()[i], dst.mutable_data()[i]);
        }
    }
};
template <typename T>
struct scalar_of {
    using type = T;
};
template <typename E, typename L>
struct scalar_of<RegTile<E, L>> {
    using type = typename scalar_of<E>::type;
};
}  // namespace detail

template <typename Tile>
using RegTileExp = detail::ElementWise<Tile, Exp<typename detail::scalar_of<Tile>::type>>;
template <typename Tile>
using RegTileLog = detail::ElementWise<Tile, Log<typename detail::scalar_of<Tile>::type>>;
template <typename Tile>
using RegTileRelu = detail::ElementWise<Tile, Relu<typename detail::scalar_of<Tile>::type>>;
template <typename Tile>
using RegTileAdd = detail::ElementWise2<Tile, Add<typename detail::scalar_of<Tile>::type>>;
template <typename Tile>
using RegTileSub = detail::ElementWise2<Tile, Sub<typename detail::scalar_of<Tile>::type>>;
template <typename Tile>
using RegTileMul = detail::ElementWise2<Tile, Mul<typename detail::scalar_of<Tile>::type>>;
template <typename Tile>
using RegTileDiv = detail::ElementWise2<Tile, Div<typename detail::scalar_of<Tile>::type>>;
template <typename Tile>
using RegTileMax = detail::ElementWise2<Tile, Max<typename detail::scalar_of<Tile>::type>>;

// BaseTile spellings of the same maps, kept for source compatibility.
template <typename Tile>
using BaseTileExp = RegTileExp<Tile>;
template <typename Tile>
using BaseTileAdd = RegTileAdd<Tile>;
template <typename Tile>
using BaseTileSub = RegTileSub<Tile>;
template <typename Tile>
using BaseTileMul = RegTileMul<Tile>;
template <typename Tile>
using BaseTileDiv = RegTileDiv<Tile>;

// Type-changing copy of a flat tile (fp32 accumulator fragment -> fp16 operand fragment and back).
template <typename SrcTile, typename DstTile>
struct RegTileConvert {
    DEVICE void operator()(const SrcTile& src, DstTile& dst) const {
        static_assert(SrcTile::kNumel == DstTile::kNumel, "tiles differ in size");
        Convert<typename SrcTile::DType, typename DstTile::DType> f;
#pragma unroll
        for (int i = 0; i < SrcTile::kNumel; ++i) f(src.data()[i], dst.mutable_data()[i]);
    }
};

}  // namespace tiledcuda::cell::compute
