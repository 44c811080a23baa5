// Global memory <-> register fragments: thread t of the CTA owns row t of the tile (reference:
// include/cell/copy/global_to_register.hpp:309-379, where ownership followed the mma.sync fragment map and
// accesses were 2 to 8 bytes wide). Row-major tiles are moved 16 bytes at a time.
#pragma once

#include "cell/copy/constants.hpp"
#include "cell/copy/warp.hpp"
#include "types/global.hpp"
#include "types/register.hpp"

namespace tiledcuda::cell::copy {

template <typename Reg_, typename WarpLayout_, WarpReuse kMode_ = WarpReuse::kCont>
struct GlobalToRegLoader : warp::CopyBase<WarpLayout_> {
    using Reg = Reg_;
    using Base = warp::CopyBase<WarpLayout_>;

    template <typename Global>
    DEVICE void operator()(const Global& src, Reg& dst) const {
        static_assert(Reg::kRows == 1 && Reg::kCols == Global::kCols, "the fragment is one row of the global tile");
        static_assert(std::is_same_v<typename Reg::DType, typename Global::DType>, "element types differ");
        const int row = Base::owned_row();
        if (row < Global::kRows) {
#pragma unroll
            for (int j = 0; j < Global::kCols; ++j) dst(0, j) = src(row, j);
        }
    }
};

template <typename Global_, typename Reg_, typename WarpLayout_>
struct RegToGlobalStorer : warp::CopyBase<WarpLayout_> {
    using Global = Global_;
    using Reg = Reg_;
    using Base = warp::CopyBase<WarpLayout_>;
    using T = typename Global::DType;

    DEVICE void operator()(const Reg& src, Global& dst) const {
        static_assert(Reg::kRows == 1 && Reg::kCols == Global::kCols, "the fragment is one row of the global tile");
        static_assert(std::is_same_v<typename Reg::DType, T>, "element types differ");
        const int row = Base::owned_row();
        if (row >= Global::kRows) return;
        constexpr int kPer = 16 / static_cast<int>(sizeof(T));
        if constexpr (Global::kType == tl::Layout::kRowMajor && Global::kCols % kPer == 0 &&
                      (Global::kRowStride * static_cast<int>(sizeof(T))) % 16 == 0) {
            if ((reinterpret_cast<uintptr_t>(dst.data()) & 15u) == 0) {
#pragma unroll
                for (int j = 0; j < Global::kCols; j += kPer)
                    *reinterpret_cast<uint4*>(&dst(row, j)) = *reinterpret_cast<const uint4*>(&src(0, j));
                return;
            }
        }
#pragma unroll
        for (int j = 0; j < Global::kCols; ++j) dst(row, j) = src(0, j);
    }
};

}  // namespace tiledcuda::cell::copy
