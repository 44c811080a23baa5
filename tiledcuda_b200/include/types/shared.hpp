// SharedTile: a typed view of a tile in shared memory.
//
// The reference's SharedTile<T, Layout, kSwizzled> (include/types/shared.hpp:9-46) stores 16x16 BaseTiles
// for ldmatrix. Here a 16-bit SharedTile is an MMA operand: it is stored in the layout tcgen05.mma reads
// (tl::OperandLayout: 128-byte swizzle when kSwizzled, interleaved 8x8 core matrices otherwise), keyed on
// which extent is contiguous: a RowMajor<R, C> tile is an operand with R outer rows and K = C; a
// ColMajor<R, C> tile (the reference's B operand, K x N) is an operand with C outer rows and K = R. Both
// are "K-major" to the tensor core. Logical (row, col) indexing is unchanged for the user. A 32-bit
// SharedTile (epilogue staging) is a plain strided tile. The base address must be 1024-byte aligned for
// swizzled tiles, 128-byte aligned otherwise.
#pragma once

#include "types/layout.hpp"

namespace tiledcuda::cell {

template <typename Element_, typename Layout_, bool kSwizzled_ = false>
class SharedTile {
  public:
    using DType = Element_;
    using Layout = Layout_;

    static constexpr int kRows = tl::num_rows<Layout>;
    static constexpr int kCols = tl::num_cols<Layout>;
    static constexpr int kRowStride = tl::row_stride<Layout>;
    static constexpr int kColStride = tl::col_stride<Layout>;
    static constexpr tl::Layout kType = tl::layout_type<Layout>;
    static constexpr bool kSwizzled = kSwizzled_;
    static constexpr bool kIsOperand = sizeof(DType) == 2;  // 16-bit tiles feed the tensor core

    // Operand view: outer extent (M or N) and contiguous extent (K).
    static constexpr int kOuter = kType == tl::Layout::kRowMajor ? kRows : kCols;
    static constexpr int kK = kType == tl::Layout::kRowMajor ? kCols : kRows;
    using Operand = tl::OperandLayout<kOuter, kK, kSwizzled>;

    static constexpr int kNumel = kIsOperand ? Operand::kNumel : tl::get_numel<Layout>;
    static constexpr int kBytes = kNumel * static_cast<int>(sizeof(DType));

    HOST_DEVICE SharedTile(DType* data) : data_(data) {}

    HOST_DEVICE DType* mutable_data() { return data_; }
    HOST_DEVICE const DType* data() const { return data_; }

    // Element offset of logical (row, col) inside the tile's storage.
    HOST_DEVICE static constexpr int offset(int x, int y) {
        if constexpr (kIsOperand) {
            return kType == tl::Layout::kRowMajor ? Operand{}(x, y) : Operand{}(y, x);
        } else {
            return Layout{}(x, y);
        }
    }

    HOST_DEVICE DType& operator()(int x, int y) { return data_[offset(x, y)]; }
    HOST_DEVICE const DType& operator()(int x, int y) const { return data_[offset(x, y)]; }

    // Byte distance from data() to where the MMA descriptor of K step `k_step` (16 elements) starts: inside a
    // 128-byte swizzle row a step is 32 bytes, every fourth step moves to the next 64-element chunk; in the
    // interleaved layout a step is two 8x8 core matrices along K.
    HOST_DEVICE static constexpr int operand_offset_bytes(int k_step) {
        if constexpr (Operand::kSwizzled) {
            return (k_step >> 2) * Operand::kChunkBytes + (k_step & 3) * 32;
        } else {
            return k_step * 2 * Operand::kLbo;
        }
    }

  private:
    DType* data_;
};

}  // namespace tiledcuda::cell
