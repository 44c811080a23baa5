// Tile layouts: index -> offset maps with compile-time extents.
//
//   MatrixLayout<R, C, rs, cs>, RowMajor<R, C, ld>, ColMajor<R, C, ld>      plain strided layouts for global
//       memory and registers, as in the reference (include/types/layout.hpp:26-53);
//   OperandLayout<Rows, K, kSwizzled>                                       the shared-memory layouts that
//       TMA writes and tcgen05.mma reads for a 16-bit K-major operand: with swizzle, 64-element (128-byte)
//       K chunks of 8-row, 1024-byte atoms whose 16-byte pieces are XOR-permuted by the row; without, the
//       interleaved layout of 8x8 core matrices. They take the place of the reference's BaseTile-blocked
//       Swizzle<2,3,3> layouts (layout.hpp:58-206), which were shaped for ldmatrix;
//   SharedLayoutWrapper<Shared>::Layout                                     the storage layout of a shared tile
//       picked from its element width and kSwizzled flag, as layout.hpp:208-273 does.
// All of it is constexpr arithmetic and compiles on the host.
#pragma once

#include <cstddef>
#include <type_traits>

#include "cell/traits/base.hpp"
#include "config.hpp"

namespace tiledcuda::cell {
namespace tile_layout {

enum class Layout { kRowMajor = 0, kColMajor = 1, kSwizzledRowMajor = 2, kSwizzledColMajor = 3 };

template <int kRows_, int kCols_, int kRowStride_, int kColStride_>
struct MatrixLayout {
    static constexpr int kRows = kRows_;
    static constexpr int kCols = kCols_;
    static constexpr int kRowStride = kRowStride_;
    static constexpr int kColStride = kColStride_;
    static constexpr int kNumel = kRows * kCols;
    // A unit column stride makes a layout row-major (so does a 1x1 layout, as in the reference).
    static constexpr Layout kType = kColStride == 1 ? Layout::kRowMajor : Layout::kColMajor;

    HOST_DEVICE constexpr int operator()(int i, int j) const { return i * kRowStride + j * kColStride; }
};

template <int kRows, int kCols, int kStride = kCols>
using RowMajor = MatrixLayout<kRows, kCols, kStride, 1>;

template <int kRows, int kCols, int kStride = kRows>
using ColMajor = MatrixLayout<kRows, kCols, 1, kStride>;

template <typename L>
inline constexpr size_t num_rows = L::kRows;
template <typename L>
inline constexpr size_t num_cols = L::kCols;
template <typename L>
inline constexpr size_t row_stride = L::kRowStride;
template <typename L>
inline constexpr size_t col_stride = L::kColStride;
template <typename L>
inline constexpr size_t get_numel = L::kNumel;
template <typename L>
inline constexpr Layout layout_type = L::kType;

// Sub-tile layout that keeps the parent's strides (used by the tile iterators).
template <int kRows, int kCols, int kRowStride, int kColStride>
HOST_DEVICE constexpr auto make_tile_layout() {
    return MatrixLayout<kRows, kCols, kRowStride, kColStride>{};
}

// Shared-memory layout of a 16-bit operand whose contiguous (K) extent is kK and whose other extent is
// kOuter (rows of A, or columns of a column-major B). operator()(o, k) returns the ELEMENT offset.
template <int kOuter_, int kK_, bool kSwizzled_>
struct OperandLayout {
    static constexpr int kOuter = kOuter_;
    static constexpr int kK = kK_;
    static constexpr bool kSwizzled = kSwizzled_;
    static constexpr int kElemBytes = 2;
    static constexpr int kChunkElems = traits::Sm100::kSwizzleBytes / kElemBytes;  // 64 elements per swizzled row
    // Storage is padded to whole chunks / whole 8-row groups so that every offset the MMA unit derives stays inside.
    static constexpr int kOuterPadded = (kOuter + 7) / 8 * 8;
    static constexpr int kChunks = kSwizzled ? (kK + kChunkElems - 1) / kChunkElems : 1;
    static constexpr int kKPadded = kSwizzled ? kChunks * kChunkElems : (kK + 7) / 8 * 8;
    static constexpr int kNumel = kOuterPadded * kKPadded;
    static constexpr int kBytes = kNumel * kElemBytes;
    // Byte distances the MMA descriptor needs.
    static constexpr int kChunkBytes = kOuterPadded * traits::Sm100::kSwizzleBytes;  // between 64-wide K chunks (swizzled)
    static constexpr int kSbo = kSwizzled ? 1024 : (kKPadded / 8) * 128;             // between 8-row groups
    static constexpr int kLbo = kSwizzled ? 16 : 128;                                // between core matrices along K (plain)

    HOST_DEVICE constexpr int byte_offset(int o, int k) const {
        if constexpr (kSwizzled) {
            const int chunk = k / kChunkElems;
            const int kin = k % kChunkElems;
            const int piece = (kin / 8) ^ (o & 7);  // 16-byte piece, permuted by the row inside the atom
            return chunk * kChunkBytes + (o >> 3) * 1024 + (o & 7) * 128 + piece * 16 + (kin & 7) * kElemBytes;
        } else {
            return (o >> 3) * kSbo + (k >> 3) * kLbo + (o & 7) * 16 + (k & 7) * kElemBytes;
        }
    }
    HOST_DEVICE constexpr int operator()(int o, int k) const { return byte_offset(o, k) / kElemBytes; }
};

// Storage layout of a shared tile: the operand layout (swizzled or interleaved, by the tile's kSwizzled flag)
// for a 16-bit tile, the tile's own strided layout for a 32-bit one. For a column-major operand tile the
// operand layout is indexed (col, row): its first index is the outer (N) extent.
template <typename Shared>
struct SharedLayoutWrapper {
    static constexpr bool kIsOperand = Shared::kIsOperand;
    using Layout = std::conditional_t<kIsOperand, OperandLayout<Shared::kOuter, Shared::kK, Shared::kSwizzled>, typename Shared::Layout>;
};

}  // namespace tile_layout
namespace tl = tile_layout;
}  // namespace tiledcuda::cell
