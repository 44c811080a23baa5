// GlobalTile: a typed view of a tile in global memory with a static layout.
// Counterpart of the reference's include/types/global.hpp:9-47 (without the printf dump).
#pragma once

#include "types/layout.hpp"

namespace tiledcuda::cell {

template <typename Element_, typename Layout_>
struct GlobalTile {
    using DType = Element_;
    using Layout = Layout_;

    static constexpr int kNumel = tl::get_numel<Layout>;
    static constexpr int kRows = tl::num_rows<Layout>;
    static constexpr int kCols = tl::num_cols<Layout>;
    static constexpr int kRowStride = tl::row_stride<Layout>;
    static constexpr int kColStride = tl::col_stride<Layout>;
    static constexpr tl::Layout kType = tl::layout_type<Layout>;

    HOST_DEVICE GlobalTile(DType* data) : data_(data) {}
    HOST_DEVICE GlobalTile(const DType* data) : data_(const_cast<DType*>(data)) {}

    HOST_DEVICE DType* mutable_data() { return data_; }
    HOST_DEVICE const DType* data() const { return data_; }
    HOST_DEVICE constexpr Layout layout() const { return Layout{}; }

    HOST_DEVICE DType& operator()(int x, int y) { return data_[Layout{}(x, y)]; }
    HOST_DEVICE const DType& operator()(int x, int y) const { return data_[Layout{}(x, y)]; }

  private:
    DType* data_;
};

}  // namespace tiledcuda::cell
