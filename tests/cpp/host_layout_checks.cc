// Host-side entry points over the layout / iterator arithmetic of the tile headers (they are plain
// constexpr C++), so that the CPU test-suite can check them without a GPU. Cases follow the reference's
// host tests: tests/cpp/cell/test_layout.cu:105-136 and test_global_tile_iterator.cu:55-66, 142-154.
#include "types/mod.hpp"

using namespace tiledcuda::cell;

extern "C" {

// layout traits of RowMajor<4, 9> / ColMajor<4, 9>: rows, cols, row stride, col stride, numel, is_row_major
void tch_layout_traits(int col_major, int* out) {
    if (!col_major) {
        using L = tl::RowMajor<4, 9>;
        out[0] = tl::num_rows<L>; out[1] = tl::num_cols<L>; out[2] = tl::row_stride<L>; out[3] = tl::col_stride<L>;
        out[4] = tl::get_numel<L>; out[5] = tl::layout_type<L> == tl::Layout::kRowMajor;
    } else {
        using L = tl::ColMajor<4, 9>;
        out[0] = tl::num_rows<L>; out[1] = tl::num_cols<L>; out[2] = tl::row_stride<L>; out[3] = tl::col_stride<L>;
        out[4] = tl::get_numel<L>; out[5] = tl::layout_type<L> == tl::Layout::kRowMajor;
    }
}

// Walk a 4 x 9 tile in 2 x 3 chunks with GTileIterator; write, for chunk (i, j) and element (r, c), the
// value found through the iterator into out[((i*3 + j)*2 + r)*3 + c].
void tch_iterate_4x9(int col_major, const float* data, float* out) {
    if (!col_major) {
        using Tile = GlobalTile<float, tl::RowMajor<4, 9>>;
        GTileIterator<Tile, TileShape<2, 3>> it(data);
        for (int i = 0; i < 2; ++i)
            for (int j = 0; j < 3; ++j) {
                auto chunk = it(i, j);
                for (int r = 0; r < 2; ++r)
                    for (int c = 0; c < 3; ++c) out[((i * 3 + j) * 2 + r) * 3 + c] = chunk(r, c);
            }
    } else {
        using Tile = GlobalTile<float, tl::ColMajor<4, 9>>;
        GTileIterator<Tile, TileShape<2, 3>> it(data);
        for (int i = 0; i < 2; ++i)
            for (int j = 0; j < 3; ++j) {
                auto chunk = it(i, j);
                for (int r = 0; r < 2; ++r)
                    for (int c = 0; c < 3; ++c) out[((i * 3 + j) * 2 + r) * 3 + c] = chunk(r, c);
            }
    }
}

// Slices: row strip 1 then its chunk 2, and column strip 1 then its chunk 1, of the row-major 4 x 9 tile;
// also the single-index form on a 2 x 9 strip. Returns element (0, 0) of each.
void tch_slices(const float* data, float* out) {
    using Tile = GlobalTile<float, tl::RowMajor<4, 9>>;
    GTileIterator<Tile, TileShape<2, 3>> it(data);
    auto row_strip = it(1, _);
    out[0] = row_strip(2)(0, 0);           // rows 2.., cols 6..  -> data[2*9 + 6]
    auto col_strip = it(_, 1);
    out[1] = col_strip(1)(0, 0);           // rows 2.., cols 3..  -> data[2*9 + 3]
    out[2] = row_strip.to_tile()(1, 8);    // last element of the strip -> data[3*9 + 8]
    out[3] = static_cast<float>(decltype(it)::sc0 * 10 + decltype(it)::sc1);
    out[4] = static_cast<float>(decltype(row_strip)::sc0 * 10 + decltype(row_strip)::sc1);
}

// Operand layouts: byte offset of (outer, k) in a 128 x 128 fp16 operand tile, swizzled or interleaved.
int tch_operand_offset(int swizzled, int outer, int k) {
    if (swizzled) return tl::OperandLayout<128, 128, true>{}.byte_offset(outer, k);
    return tl::OperandLayout<128, 128, false>{}.byte_offset(outer, k);
}

// Sizes: bytes of SharedTile<half, RowMajor<64,128>, swizzled>, of SharedTile<half, ColMajor<32, 80>, plain>
// and of SharedTile<float, RowMajor<16, 24>>; numel of TileShape<64, 64, 128, 128>; dim 2 of it.
void tch_sizes(long long* out) {
    out[0] = SharedTile<unsigned short, tl::RowMajor<64, 128>, true>::kBytes;
    out[1] = SharedTile<unsigned short, tl::ColMajor<32, 80>, false>::kBytes;
    out[2] = SharedTile<float, tl::RowMajor<16, 24>, false>::kBytes;
    out[3] = get_numel<TileShape<64, 64, 128, 128>>;
    out[4] = dim_size<2, TileShape<64, 64, 128, 128>>;
    out[5] = tmem_alloc_columns(80);
    out[6] = STileIterator<SharedTile<unsigned short, tl::RowMajor<128, 128>, true>, TileShape<128, 64>>::chunk_offset(1);
    out[7] = BaseTileRowMajor<float>::kNumel;
}

// RegTile: nested clear and indexing on the host.
float tch_regtile() {
    RegTile<BaseTileRowMajor<float>, tl::RowMajor<2, 3>> t;
    t(1, 2)(1, 3) = 5.f;
    float s = t(1, 2)(1, 3);
    t.clear();
    return s + t(1, 2)(1, 3);
}

}  // extern "C"
