// Shared memory <-> register fragments.
//
// In the reference SharedToRegLoader feeds the tensor core: ldmatrix moves operand sub-tiles into
// per-warp fragments (include/cell/copy/shared_to_register.hpp:194-238). tcgen05.mma takes its operands
// from shared memory through a descriptor, so for MMA operands the "load" is make_operand_descriptor()
// and no data moves. The functors below keep the reference's names for the element-wise paths: thread t
// of the CTA owns row t (the TMEM lane rule), loads it from / stores it to a shared tile, converting
// between fp32 fragments and 16-bit tiles on the way (that is how an intermediate such as fp16(A B)
// becomes the A operand of a second MMA without leaving the chip).
#pragma once

#include <cstdint>

#include "cell/copy/constants.hpp"
#include "cell/copy/warp.hpp"
#include "types/register.hpp"
#include "types/shared.hpp"

namespace tiledcuda::cell::copy {

// 64-bit shared-memory matrix descriptor of a 16-bit operand tile (a SharedTile, or a chunk of one from an
// STileIterator) for tcgen05.mma; `k_step` selects the 16-element K step inside it.
template <typename Shared>
DEVICE uint64_t make_operand_descriptor(const Shared& tile, int k_step = 0) {
    static_assert(Shared::kIsOperand, "only 16-bit shared tiles are MMA operands");
    using Op = typename Shared::Operand;
    // a whole SharedTile starts at data(); a chunk handed out by an STileIterator starts inside its parent
    const uint32_t addr = static_cast<uint32_t>(__cvta_generic_to_shared(tile.data())) +
                          static_cast<uint32_t>(tile.operand_offset_bytes(k_step));
    uint64_t d = 0;
    d |= static_cast<uint64_t>((addr & 0x3ffffu) >> 4);
    d |= static_cast<uint64_t>((Op::kLbo >> 4) & 0x3fff) << 16;
    d |= static_cast<uint64_t>((Op::kSbo >> 4) & 0x3fff) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(Op::kSwizzled ? 2 : 0) << 61;
    return d;
}

namespace detail {
template <typename To, typename From>
DEVICE To convert(From v) {
    if constexpr (std::is_same_v<To, From>) {
        return v;
    } else if constexpr (std::is_same_v<To, __half>) {
        return __float2half(static_cast<float>(v));
    } else {
        return static_cast<To>(__half2float(v));
    }
}
}  // namespace detail

// shared tile row (threadIdx-owned) -> RowFragment
template <typename Reg_, typename WarpLayout_, WarpReuse kMode_ = WarpReuse::kCont>
struct SharedToRegLoader : warp::CopyBase<WarpLayout_> {
    using Reg = Reg_;
    using Base = warp::CopyBase<WarpLayout_>;

    template <typename Shared>
    DEVICE void operator()(const Shared& src, Reg& dst) const {
        static_assert(Reg::kRows == 1 && Reg::kCols == Shared::kCols, "the fragment is one row of the shared tile");
        const int row = Base::owned_row();
        if (row < Shared::kRows) {
#pragma unroll
            for (int j = 0; j < Shared::kCols; ++j) dst(0, j) = detail::convert<typename Reg::DType>(src(row, j));
        }
    }
};

// RowFragment -> shared tile row, converting to the tile's element type
template <typename Reg_, typename WarpLayout_>
struct RegToSharedStorer : warp::CopyBase<WarpLayout_> {
    using Reg = Reg_;
    using Base = warp::CopyBase<WarpLayout_>;

    template <typename Shared>
    DEVICE void operator()(const Reg& src, Shared& dst) const {
        static_assert(Reg::kRows == 1 && Reg::kCols == Shared::kCols, "the fragment is one row of the shared tile");
        using T = typename Shared::DType;
        const int row = Base::owned_row();
        if (row < Shared::kRows) {
            if constexpr (sizeof(T) == 2 && Shared::kType == tl::Layout::kRowMajor && Shared::kCols % 8 == 0) {
                // eight 16-bit elements are one 16-byte piece of the operand layout
#pragma unroll
                for (int j = 0; j < Shared::kCols; j += 8) {
                    alignas(16) T piece[8];
#pragma unroll
                    for (int e = 0; e < 8; ++e) piece[e] = detail::convert<T>(src(0, j + e));
                    *reinterpret_cast<uint4*>(dst.mutable_data() + Shared::offset(row, j)) = *reinterpret_cast<const uint4*>(piece);
                }
            } else {
#pragma unroll
                for (int j = 0; j < Shared::kCols; ++j) dst(row, j) = detail::convert<T>(src(0, j));
            }
        }
    }
};

}  // namespace tiledcuda::cell::copy
