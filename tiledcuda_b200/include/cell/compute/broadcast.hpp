// Broadcasts of a per-row value over a register tile (reference: include/cell/compute/broadcast.hpp:11-160).
// With one row per thread the "vector" is a single scalar per thread: dst(0, j) = f(dst(0, j), vec).
#pragma once

#include "cell/compute/math_functor.hpp"
#include "types/register.hpp"

namespace tiledcuda::cell::compute {

template <typename SrcVec, typename DstTile, tl::Layout kLayout = tl::Layout::kRowMajor>
struct Broadcast {
    DEVICE void operator()(const SrcVec& src, DstTile& dst) const {
        static_assert(SrcVec::kNumel == 1 && DstTile::kRows == 1, "one row and one row value per thread");
#pragma unroll
        for (int j = 0; j < DstTile::kCols; ++j) dst(0, j) = src(0, 0);
    }
};

namespace detail {
template <typename SrcVec, typename DstTile, typename Functor>
struct BroadcastOp {
    DEVICE void operator()(const SrcVec& vec, DstTile& dst) const {
        static_assert(SrcVec::kNumel == 1 && DstTile::kRows == 1, "one row and one row value per thread");
        Functor f;
        const typename DstTile::DType v = vec(0, 0);
#pragma unroll
        for (int j = 0; j < DstTile::kCols; ++j) dst(0, j) = f(dst(0, j), v);
    }
};
}  // namespace detail

template <typename SrcVec, typename DstTile, tl::Layout kLayout = tl::Layout::kRowMajor>
using BroadcastAdd = detail::BroadcastOp<SrcVec, DstTile, Add<typename DstTile::DType>>;
template <typename SrcVec, typename DstTile, tl::Layout kLayout = tl::Layout::kRowMajor>
using BroadcastSub = detail::BroadcastOp<SrcVec, DstTile, Sub<typename DstTile::DType>>;
template <typename SrcVec, typename DstTile, tl::Layout kLayout = tl::Layout::kRowMajor>
using BroadcastMul = detail::BroadcastOp<SrcVec, DstTile, Mul<typename DstTile::DType>>;
template <typename SrcVec, typename DstTile, tl::Layout kLayout = tl::Layout::kRowMajor>
using BroadcastDiv = detail::BroadcastOp<SrcVec, DstTile, Div<typename DstTile::DType>>;

}  // namespace tiledcuda::cell::compute
