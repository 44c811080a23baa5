"""CPU tests of the C-ABI boundary: the library loads without a GPU, exports every symbol that
include/tiledcuda_b200.h declares, and rejects bad arguments with a status and a message before it
touches CUDA. No compute call is made here."""
import ctypes
import re
from pathlib import Path

import pytest

from tiledcuda_b200 import _lib

ROOT = Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "tiledcuda_b200.h"


def declared_symbols():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(tc_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    names = declared_symbols()
    for want in ("tc_gemm_f16_f32", "tc_gemm_bf16_f32", "tc_gemm_f16_f32_host", "tc_gemm_tile_plan", "tc_lstm_chain_ws_f16", "tc_lstm_chain_static_f16", "tc_b2b_gemm_f16", "tc_flash_attn_fwd_f16", "tc_flash_attn_fwd_ex_f16", "tc_scatter_nd_add", "tc_lstm_cell_f16",
                 "tc_lstm_chain_f16", "tc_scatter_nd", "tc_last_error", "tc_device_status", "tc_version"):
        assert want in names


def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(str(_lib.LIB_PATH))
    for name in declared_symbols():
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"


def test_python_binding_covers_every_declared_symbol():
    assert sorted(_lib.SIGNATURES) == declared_symbols()
    assert _lib.load().tc_version() >= 1000


def test_every_declaration_cites_the_reference_or_says_it_has_no_counterpart():
    text = HEADER.read_text()
    for m in re.finditer(r"/\*(.*?)\*/\s*(?:int|const char\*)\s+(tc_[a-z0-9_]+)\s*\(", text, flags=re.S):
        comment, name = m.group(1), m.group(2)
        if name in ("tc_last_error", "tc_version"):
            continue
        assert re.search(r"\.(cu|hpp|py|cc)?:?\d+|Makefile:\d+|no counterpart", comment), name


@pytest.mark.parametrize(
    "call, needle",
    [
        (lambda l: l.tc_gemm_f16_f32(None, None, None, 128, 128, 64, 64, 64, 128, None), "null"),
        (lambda l: l.tc_gemm_f16_f32(16, 16, 16, 128, 128, 60, 64, 64, 128, None), "multiple of 8"),
        (lambda l: l.tc_gemm_f16_f32(16, 16, 16, 0, 128, 64, 64, 64, 128, None), "positive"),
        (lambda l: l.tc_gemm_f16_f32(16, 16, 16, 128, 128, 64, 32, 64, 128, None), "leading dimension"),
        (lambda l: l.tc_gemm_f16_f32(18, 16, 16, 128, 128, 64, 64, 64, 128, None), "aligned"),
        (lambda l: l.tc_b2b_gemm_f16(16, 16, 16, 16, 128, 128, 256, 128, 1, None), "[16,128]"),
        (lambda l: l.tc_b2b_gemm_f16(16, 16, 16, 16, 128, 100, 128, 128, 1, None), "multiple of 8"),
        (lambda l: l.tc_flash_attn_fwd_f16(16, 16, 16, 16, None, 1, 1, 128, 128, 72, 128, 1.0, 0, None), "multiple of 16"),
        (lambda l: l.tc_flash_attn_fwd_f16(16, 16, 16, 16, None, 0, 1, 128, 128, 64, 64, 1.0, 0, None), "positive"),
        (lambda l: l.tc_flash_attn_fwd_f16(16, 16, 16, 16, None, 1, 1, 128, 128, 64, 64, float("nan"), 0, None), "finite"),
        (lambda l: l.tc_lstm_cell_f16(16, 16, None, 16, 16, 16, 16, 16, 8, 64, 24, None), "multiple of 16"),
        (lambda l: l.tc_lstm_cell_f16(16, 16, None, 16, 32, 16, 32, 16, 8, 64, 32, None), "alias"),
        (lambda l: l.tc_lstm_chain_f16(16, 16, None, 16, 16, 16, 16, 16, 0, 8, 64, 32, None), "steps"),
        (lambda l: l.tc_lstm_chain_static_f16(16, 16, None, 16, 16, 16, 16, 16, -1, 8, 64, 32, None), "negative"),
    ],
)
def test_bad_arguments_return_a_status_and_a_message(call, needle):
    lib = _lib.load()
    rc = call(lib)
    assert rc == -1  # TC_ERR_BAD_ARG
    assert needle in lib.tc_last_error().decode()


def test_static_chain_refuses_sizes_beyond_its_built_in_scratch_without_a_device():
    """The 64 MiB limit is tested by division: a step count that would wrap steps * batch * 4 * hidden * 4 around
    2^64 is refused like any other oversize request, before any device is touched."""
    lib = _lib.load()
    for steps in (1 << 62, (1 << 64) // (8 * 4 * 32 * 4) + 1, 1 << 40, 16385):
        rc = lib.tc_lstm_chain_static_f16(16, 16, None, 16, 16, 16, 16, 16, steps % (1 << 63), 8, 64, 32, None)
        assert rc == -2, steps  # TC_ERR_UNSUPPORTED
        assert "built into" in lib.tc_last_error().decode()


def test_peer_window_and_sm_budget_argument_checks():
    lib = _lib.load()
    buf = ctypes.create_string_buffer(64)
    assert lib.tc_peer_export(None, buf, 64) == -1 and "null" in lib.tc_last_error().decode()
    assert lib.tc_peer_export(16, buf, 8) == -1 and "handle buffer" in lib.tc_last_error().decode()
    out = ctypes.c_void_p()
    assert lib.tc_peer_open(buf, 8, ctypes.byref(out)) == -1
    assert lib.tc_peer_copy(None, 16, 4, None) == -1
    assert lib.tc_peer_close(None) == 0
    assert lib.tc_gemm_f16_f32_sms(16, 16, 16, 128, 128, 64, 64, 64, 128, -3, None) == -1 and "max_sms" in lib.tc_last_error().decode()
    assert lib.tc_gemm_f16_f32_sms(16, 16, 16, 128, 128, 64, 64, 64, 128, 1, None) == -1


def test_scatter_argument_checks():
    lib = _lib.load()
    dims = (ctypes.c_int64 * 2)(8, 4)
    assert lib.tc_scatter_nd(None, 16, 16, 0, dims, 2, 4, 1, 2, None) == -1
    assert lib.tc_scatter_nd(16, 16, 16, 0, dims, 2, 4, 3, 2, None) == -1  # k > rank
    assert lib.tc_scatter_nd(16, 16, 16, 0, dims, 2, 4, 1, 3, None) == -1  # elem_bytes
    assert "elem_bytes" in lib.tc_last_error().decode()
    assert lib.tc_scatter_nd(16, 16, 16, 0, dims, 2, 0, 1, 2, None) == 0   # n == 0: nothing to do


def test_check_raises_with_the_library_message():
    lib = _lib.load()
    rc = lib.tc_gemm_f16_f32(None, None, None, 1, 1, 8, 8, 8, 1, None)
    with pytest.raises(_lib.TiledCudaError) as ei:
        _lib.check("tc_gemm_f16_f32", rc)
    assert ei.value.status == -1 and "null" in str(ei.value)


def test_gemm_tile_plan_is_a_pure_function_and_parity_shapes_cover_every_tile():
    """tc_gemm_tile_plan needs no GPU. The headline size takes the tall pair tiles, mid sizes the square pair
    tiles, small ones lone CTAs (128x64 tiles while 128x128 ones would leave half the SMs idle); and the GEMM
    shapes of the GPU parity suite reach all five kernels."""
    lib = _lib.load()
    plan = lambda m, n, k: lib.tc_gemm_tile_plan(m, n, k, 148)
    assert plan(8192, 8192, 8192) == 3 and plan(16384, 16384, 16384) == 3
    assert plan(4096, 4096, 4096) == 2 and plan(2048, 2048, 2048) == 2 and plan(8192, 8192, 2048) == 2
    assert plan(1024, 1024, 1024) == 4 and plan(16, 16, 16) == 4 and plan(100000, 64, 512) == 4
    assert plan(1536, 1536, 1536) == 0 and plan(2304, 2304, 64) == 0
    assert plan(128, 19200, 256) == 1
    assert lib.tc_gemm_tile_plan(0, 8, 8, 148) == -1 and lib.tc_gemm_tile_plan(8, 8, 8, 0) == -1
    from tests.test_gpu_parity import GEMM_SHAPES
    kinds = {plan(*shape) for shape in GEMM_SHAPES} | {plan(16384 + 328, 16384 - 56, 8192)}  # + the tall-tile test
    assert kinds == {0, 1, 2, 3, 4}
