// STileIterator: walks a shared-memory operand tile in chunks and hands out views that compute::gemm
// accepts as MMA operands, so that a kernel can load a wide K slab once and multiply it in narrower steps:
//
//     for (int k2 = 0; k2 < SIterA::sc1; ++k2) compute::gemm(sAs(k2), sBs(k2), acc, ...);
//
// Counterpart of the reference's include/types/shared_tile_iterator.hpp:31-129, which likewise implements
// only the single-index form (its chunks go to SharedToRegLoader and from there to gemm; here they go to
// gemm directly, because tcgen05.mma reads its operands from shared memory).
//
// A chunk is NOT a relocated copy of the operand layout: inside a 128-byte swizzle row the 16-byte pieces
// are permuted by the row index, so a chunk that starts mid-row is still addressed through the parent's
// layout. SharedTileChunk therefore keeps the parent's base pointer and strides and only records where the
// chunk starts. Chunk extents must respect what the tensor core can address: a K extent that is a multiple
// of 16 elements and an outer extent that is a multiple of 8 rows.
#pragma once

#include "types/shared.hpp"
#include "types/tile_shape.hpp"

namespace tiledcuda::cell {

// A kRows x kCols window of a parent SharedTile, starting at logical (row0, col0).
template <class Parent_, int kRows_, int kCols_>
class SharedTileChunk {
  public:
    using Parent = Parent_;
    using DType = typename Parent::DType;
    using Operand = typename Parent::Operand;   // strides (kSbo, kLbo, kChunkBytes) are the parent's

    static constexpr int kRows = kRows_;
    static constexpr int kCols = kCols_;
    static constexpr tl::Layout kType = Parent::kType;
    static constexpr bool kSwizzled = Parent::kSwizzled;
    static constexpr bool kIsOperand = Parent::kIsOperand;
    static constexpr int kOuter = kType == tl::Layout::kRowMajor ? kRows : kCols;
    static constexpr int kK = kType == tl::Layout::kRowMajor ? kCols : kRows;
    static_assert(!kIsOperand || (kK % 16 == 0 && kOuter % 8 == 0),
                  "operand chunks span whole K steps of 16 and whole 8-row groups");

    HOST_DEVICE SharedTileChunk(DType* base, int row0, int col0) : base_(base), row0_(row0), col0_(col0) {}

    // The parent's storage; element (x, y) of the chunk lives at data()[offset(x, y)].
    HOST_DEVICE DType* mutable_data() { return base_; }
    HOST_DEVICE const DType* data() const { return base_; }
    HOST_DEVICE int row0() const { return row0_; }
    HOST_DEVICE int col0() const { return col0_; }

    HOST_DEVICE int offset(int x, int y) const { return Parent::offset(row0_ + x, col0_ + y); }
    HOST_DEVICE DType& operator()(int x, int y) { return base_[offset(x, y)]; }
    HOST_DEVICE const DType& operator()(int x, int y) const { return base_[offset(x, y)]; }

    // Byte distance from data() to where the MMA descriptor of K step `k_step` (16 elements) of this chunk
    // starts: the chunk's first 8-row group, plus its first K step, plus k_step, in the parent's strides.
    HOST_DEVICE int operand_offset_bytes(int k_step) const {
        const int outer0 = kType == tl::Layout::kRowMajor ? row0_ : col0_;
        const int k0 = kType == tl::Layout::kRowMajor ? col0_ : row0_;
        return (outer0 >> 3) * Operand::kSbo + Parent::operand_offset_bytes(k0 / 16 + k_step);
    }

  private:
    DType* base_;
    int row0_;
    int col0_;
};

template <class Tile_, class ChunkShape_>
class STileIterator {
  public:
    using Tile = Tile_;
    using DType = typename Tile::DType;
    using ChunkShape = ChunkShape_;

    static constexpr int kStride0 = dim_size<0, ChunkShape>;
    static constexpr int kStride1 = dim_size<1, ChunkShape>;
    static_assert(Tile::kRows % kStride0 == 0 && Tile::kCols % kStride1 == 0, "chunks must tile the tile exactly");
    static constexpr int sc0 = Tile::kRows / kStride0;
    static constexpr int sc1 = Tile::kCols / kStride1;
    static_assert(sc0 == 1 || sc1 == 1, "shared tiles are chunked along one dimension");

    using Chunk = SharedTileChunk<Tile, kStride0, kStride1>;

    HOST_DEVICE STileIterator() : data_(nullptr) {}
    HOST_DEVICE STileIterator(DType* data) : data_(data) {}
    HOST_DEVICE STileIterator(Tile& tile) : data_(tile.mutable_data()) {}

    // Storage offset (elements) of the first element of chunk i.
    HOST_DEVICE static constexpr int chunk_offset(int i) {
        return sc0 == 1 ? Tile::offset(0, i * kStride1) : Tile::offset(i * kStride0, 0);
    }

    HOST_DEVICE Chunk operator()(int i) const {
        return sc0 == 1 ? Chunk(data_, 0, i * kStride1) : Chunk(data_, i * kStride0, 0);
    }

    HOST_DEVICE Tile to_tile() const { return Tile(data_); }

  private:
    DType* data_;
};

}  // namespace tiledcuda::cell
