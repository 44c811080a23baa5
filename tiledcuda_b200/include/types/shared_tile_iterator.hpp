// STileIterator: walks a shared-memory operand tile along K in chunks; returns SharedTile views whose
// storage offsets follow the operand layout (so a chunk is directly usable by compute::gemm).
// Counterpart of the reference's include/types/shared_tile_iterator.hpp:31-129, which likewise implements
// only the single-index form.
#pragma once

#include "types/shared.hpp"
#include "types/tile_shape.hpp"

namespace tiledcuda::cell {

template <class Tile_, class ChunkShape_>
class STileIterator {
  public:
    using Tile = Tile_;
    using DType = typename Tile::DType;
    using ChunkShape = ChunkShape_;

    static constexpr int kStride0 = dim_size<0, ChunkShape>;
    static constexpr int kStride1 = dim_size<1, ChunkShape>;
    static constexpr int sc0 = Tile::kRows / kStride0;
    static constexpr int sc1 = Tile::kCols / kStride1;
    static_assert(sc0 == 1 || sc1 == 1, "shared tiles are chunked along one dimension (K)");

    HOST_DEVICE STileIterator() : data_(nullptr) {}
    HOST_DEVICE STileIterator(DType* data) : data_(data) {}

    // Storage offset (elements) of the first element of chunk i.
    HOST_DEVICE static constexpr int chunk_offset(int i) {
        return sc0 == 1 ? Tile::offset(0, i * kStride1) : Tile::offset(i * kStride0, 0);
    }

    // The chunk keeps the parent's storage layout: it is addressed through the parent, starting at the
    // chunk's first logical row / column.
    struct Chunk {
        DType* base;
        int row0;
        int col0;
        static constexpr int kRows = kStride0;
        static constexpr int kCols = kStride1;
        HOST_DEVICE DType& operator()(int x, int y) { return base[Tile::offset(row0 + x, col0 + y)]; }
        HOST_DEVICE const DType& operator()(int x, int y) const { return base[Tile::offset(row0 + x, col0 + y)]; }
    };

    HOST_DEVICE Chunk operator()(int i) const {
        return sc0 == 1 ? Chunk{data_, 0, i * kStride1} : Chunk{data_, i * kStride0, 0};
    }

  private:
    DType* data_;
};

}  // namespace tiledcuda::cell
