"""CPU tests of the C++ tile vocabulary (tiledcuda_b200/include/types): layouts, tile shapes, iterators
and the shared-memory operand layouts are constexpr arithmetic, compiled for the host into
tests/cpp/libhost_layout_checks.so. Cases follow the reference's host-side unit tests
(tests/cpp/cell/test_layout.cu:105-136, test_global_tile_iterator.cu:55-66, 142-154)."""
import ctypes
from pathlib import Path

import numpy as np
import pytest

LIB = Path(__file__).resolve().parent / "cpp" / "libhost_layout_checks.so"


@pytest.fixture(scope="module")
def lib():
    if not LIB.exists():
        from tiledcuda_b200 import build

        build.build_tile_api_tests()
    return ctypes.CDLL(str(LIB))


def test_layout_traits(lib):
    out = (ctypes.c_int * 6)()
    lib.tch_layout_traits(0, out)
    assert list(out) == [4, 9, 9, 1, 36, 1]   # RowMajor<4, 9>
    lib.tch_layout_traits(1, out)
    assert list(out) == [4, 9, 1, 4, 36, 0]   # ColMajor<4, 9>


@pytest.mark.parametrize("col_major", [0, 1])
def test_global_tile_iterator_chunks(lib, col_major):
    logical = np.arange(36, dtype=np.float32).reshape(4, 9)
    stored = np.ascontiguousarray(logical.T if col_major else logical).ravel()
    out = np.zeros(36, dtype=np.float32)
    lib.tch_iterate_4x9(col_major, stored.ctypes.data_as(ctypes.c_void_p), out.ctypes.data_as(ctypes.c_void_p))
    got = out.reshape(2, 3, 2, 3)
    for i in range(2):
        for j in range(3):
            assert np.array_equal(got[i, j], logical[2 * i:2 * i + 2, 3 * j:3 * j + 3])


def test_global_tile_iterator_slices(lib):
    data = np.arange(36, dtype=np.float32)
    out = np.zeros(5, dtype=np.float32)
    lib.tch_slices(data.ctypes.data_as(ctypes.c_void_p), out.ctypes.data_as(ctypes.c_void_p))
    assert out.tolist() == [2 * 9 + 6, 2 * 9 + 3, 3 * 9 + 8, 23.0, 13.0]


def test_swizzled_operand_layout_is_a_permutation_within_atoms(lib):
    lib.tch_operand_offset.restype = ctypes.c_int
    seen = set()
    for outer in range(128):
        for k in range(0, 128, 8):
            off = lib.tch_operand_offset(1, outer, k)
            assert off % 16 == 0
            chunk, rest = divmod(off, 128 * 128)          # 64-wide K chunks are 16 KiB apart for 128 rows
            assert chunk == k // 64
            atom, in_atom = divmod(rest, 1024)            # 8-row atoms
            assert atom == outer // 8
            row, piece = divmod(in_atom, 128)
            assert row == outer % 8 and piece // 16 == ((k % 64) // 8) ^ (outer % 8)
            seen.add(off)
    assert len(seen) == 128 * 16
    assert lib.tch_operand_offset(1, 5, 11) == lib.tch_operand_offset(1, 5, 8) + 6   # elements stay in order inside a piece


def test_interleaved_operand_layout(lib):
    lib.tch_operand_offset.restype = ctypes.c_int
    # 8x8 core matrices of 128 bytes: K neighbours 128 bytes apart, 8-row groups (128/8)*128 bytes apart
    assert lib.tch_operand_offset(0, 0, 0) == 0
    assert lib.tch_operand_offset(0, 0, 8) == 128
    assert lib.tch_operand_offset(0, 1, 0) == 16
    assert lib.tch_operand_offset(0, 8, 0) == 16 * 128
    assert lib.tch_operand_offset(0, 9, 17) == 16 * 128 + 2 * 128 + 16 + 2
    offs = {lib.tch_operand_offset(0, o, k) for o in range(128) for k in range(128)}
    assert len(offs) == 128 * 128 and max(offs) == 128 * 128 * 2 - 2


def test_sizes_and_shapes(lib):
    out = (ctypes.c_longlong * 8)()
    lib.tch_sizes(out)
    assert out[0] == 64 * 128 * 2          # swizzled 64 x 128 fp16
    assert out[1] == 80 * 32 * 2           # column-major 32 x 80: outer 80, K 32
    assert out[2] == 16 * 24 * 4
    assert out[3] == 64 * 64 * 128 * 128 and out[4] == 128
    assert out[5] == 128                   # TMEM allocations are powers of two >= 32 columns
    assert out[6] == 128 * 64              # second 64-wide K chunk of a swizzled 128 x 128 tile, in elements
    assert out[7] == 8


def test_regtile_nested_clear(lib):
    lib.tch_regtile.restype = ctypes.c_float
    assert lib.tch_regtile() == 5.0
