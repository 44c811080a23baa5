// Register-to-register copies (reference: include/cell/copy/register.hpp:33-38).
#pragma once

#include "types/register.hpp"

namespace tiledcuda::cell::copy {

template <typename Src, typename Dst>
DEVICE void copy(const Src& src, Dst& dst) {
    static_assert(Src::kNumel == Dst::kNumel, "fragments differ in size");
    for (int i = 0; i < Src::kNumel; ++i) dst.mutable_data()[i] = src.data()[i];
}

template <typename Element>
struct BaseTileCopy {
    DEVICE void operator()(const BaseTileRowMajor<Element>& src, BaseTileRowMajor<Element>& dst) const { copy(src, dst); }
};

template <typename Tile>
struct RegTileCopy {
    DEVICE void operator()(const Tile& src, Tile& dst) const { copy(src, dst); }
};

}  // namespace tiledcuda::cell::copy
