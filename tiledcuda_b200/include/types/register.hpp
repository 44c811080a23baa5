// RegTile: a per-thread fragment held in registers, possibly nested (a RegTile of RegTiles).
//
// The reference's fragments follow mma.sync ownership: BaseTileRowMajor = RegTile<T, RowMajor<2,4>> is the
// 8 elements one thread holds of a 16x16 BaseTile (include/types/register.hpp:65-112). tcgen05 accumulators
// live in TMEM instead, and `tcgen05.ld 32x32b` hands every thread ONE ROW of the tile: thread t of a
// 128-thread CTA owns row t, all columns. So the natural fragment here is RegTile<T, RowMajor<1, N>> (see
// RowFragment below), row reductions are thread-local, and no shuffle is needed for softmax statistics.
// The BaseTile aliases are kept so that declarations written against the reference still compile; they
// are plain 2x4 / 4x2 arrays with no hardware meaning on this architecture.
#pragma once

#include <type_traits>

#include "types/layout.hpp"

namespace tiledcuda::cell {

namespace detail {
template <typename T>
struct is_reg_tile : std::false_type {};
}  // namespace detail

template <typename Element_, typename Layout_>
class RegTile {
  public:
    using DType = Element_;
    using Layout = Layout_;

    static constexpr int kNumel = tl::get_numel<Layout>;
    static constexpr int kRows = tl::num_rows<Layout>;
    static constexpr int kCols = tl::num_cols<Layout>;
    static constexpr tl::Layout kType = tl::layout_type<Layout>;

    HOST_DEVICE RegTile() {
        for (int i = 0; i < kNumel; ++i) data_[i] = DType{};
    }

    HOST_DEVICE DType* mutable_data() { return data_; }
    HOST_DEVICE const DType* data() const { return data_; }
    HOST_DEVICE constexpr Layout layout() const { return Layout{}; }

    HOST_DEVICE DType& operator()(int x, int y) { return data_[Layout{}(x, y)]; }
    HOST_DEVICE const DType& operator()(int x, int y) const { return data_[Layout{}(x, y)]; }

    // Zero every element, recursing into nested tiles.
    HOST_DEVICE void clear() {
        for (int i = 0; i < kNumel; ++i) {
            if constexpr (detail::is_reg_tile<DType>::value)
                data_[i].clear();
            else
                data_[i] = DType{};
        }
    }

  private:
    DType data_[kNumel];
};

namespace detail {
template <typename E, typename L>
struct is_reg_tile<RegTile<E, L>> : std::true_type {};
}  // namespace detail

template <typename Element>
using BaseTileRowMajor = RegTile<Element, tl::RowMajor<2, 4>>;
template <typename Element>
using BaseTileColMajor = RegTile<Element, tl::ColMajor<4, 2>>;

// The fragment tcgen05.ld produces: the thread's row of an M x N tile.
template <typename Element, int kCols>
using RowFragment = RegTile<Element, tl::RowMajor<1, kCols>>;

// Per-row scalars (running max / sum of a softmax): one value per thread.
template <typename Element>
using RowScalar = RegTile<Element, tl::RowMajor<1, 1>>;

}  // namespace tiledcuda::cell
