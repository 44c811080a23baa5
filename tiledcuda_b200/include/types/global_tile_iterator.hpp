// GTileIterator: walks a GlobalTile in chunks of a fixed shape; pointer arithmetic only.
// Counterpart of the reference's include/types/global_tile_iterator.hpp:29-152, same indexing rules:
//   it(i)      the i-th chunk when one of the two strip counts is 1
//   it(i, j)   chunk (i, j)
//   it(i, _)   row strip i as a new iterator over its chunks;  it(_, j) likewise for a column strip
//   to_tile()  the whole iterated region as one tile
#pragma once

#include "types/global.hpp"
#include "types/tile_shape.hpp"

namespace tiledcuda::cell {

template <class Tile_, class ChunkShape_>
class GTileIterator {
  public:
    using Tile = Tile_;
    using DType = typename Tile::DType;
    using ChunkShape = ChunkShape_;

    static constexpr int kStride0 = dim_size<0, ChunkShape>;
    static constexpr int kStride1 = dim_size<1, ChunkShape>;
    static_assert(Tile::kRows >= kStride0 && Tile::kCols >= kStride1, "a chunk must fit in the tile");
    static_assert(Tile::kRows % kStride0 == 0 && Tile::kCols % kStride1 == 0, "chunks must tile the tile exactly");

    static constexpr int sc0 = Tile::kRows / kStride0;  // strips along rows
    static constexpr int sc1 = Tile::kCols / kStride1;  // strips along columns

    using ChunkLayout = tl::MatrixLayout<kStride0, kStride1, Tile::kRowStride, Tile::kColStride>;
    using Chunk = GlobalTile<DType, ChunkLayout>;

    HOST_DEVICE GTileIterator() : data_(nullptr) {}
    HOST_DEVICE GTileIterator(DType* data) : data_(data) {}
    HOST_DEVICE GTileIterator(const DType* data) : data_(const_cast<DType*>(data)) {}

    // Element offset of chunk (x, y) from the start of the tile.
    HOST_DEVICE static constexpr int chunk_offset(int x, int y) {
        return x * kStride0 * Tile::kRowStride + y * kStride1 * Tile::kColStride;
    }

    HOST_DEVICE Chunk operator()(int i) const {
        static_assert(sc0 == 1 || sc1 == 1, "a single index needs one strip count to be 1");
        return sc0 == 1 ? Chunk(data_ + chunk_offset(0, i)) : Chunk(data_ + chunk_offset(i, 0));
    }

    HOST_DEVICE Chunk operator()(int x, int y) const { return Chunk(data_ + chunk_offset(x, y)); }

    HOST_DEVICE auto operator()(int x, const Underscore&) const {
        using StripLayout = tl::MatrixLayout<kStride0, Tile::kCols, Tile::kRowStride, Tile::kColStride>;
        using Strip = GlobalTile<DType, StripLayout>;
        return GTileIterator<Strip, ChunkShape>(data_ + chunk_offset(x, 0));
    }

    HOST_DEVICE auto operator()(const Underscore&, int y) const {
        using StripLayout = tl::MatrixLayout<Tile::kRows, kStride1, Tile::kRowStride, Tile::kColStride>;
        using Strip = GlobalTile<DType, StripLayout>;
        return GTileIterator<Strip, ChunkShape>(data_ + chunk_offset(0, y));
    }

    HOST_DEVICE Tile to_tile() const { return Tile(data_); }

  private:
    DType* data_;
};

}  // namespace tiledcuda::cell
