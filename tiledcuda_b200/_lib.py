"""ctypes binding of libtiledcuda_b200.so (the C ABI declared in include/tiledcuda_b200.h).

The library is loaded from this package directory. There is no fallback: if it is missing, or a call
returns a non-zero status, an exception is raised.
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path

_PKG = Path(__file__).resolve().parent
LIB_PATH = _PKG / "libtiledcuda_b200.so"

c_i64 = ctypes.c_int64
c_vp = ctypes.c_void_p

# name -> (restype, argtypes); mirrors include/tiledcuda_b200.h one to one.
SIGNATURES = {
    "tc_last_error": (ctypes.c_char_p, []),
    "tc_version": (ctypes.c_int, []),
    "tc_device_status": (ctypes.c_int, [ctypes.POINTER(ctypes.c_int)]),
    "tc_gemm_f16_f32": (ctypes.c_int, [c_vp, c_vp, c_vp, c_i64, c_i64, c_i64, c_i64, c_i64, c_i64, c_vp]),
    "tc_gemm_bf16_f32": (ctypes.c_int, [c_vp, c_vp, c_vp, c_i64, c_i64, c_i64, c_i64, c_i64, c_i64, c_vp]),
    "tc_gemm_f16_f32_sms": (ctypes.c_int, [c_vp, c_vp, c_vp, c_i64, c_i64, c_i64, c_i64, c_i64, c_i64, ctypes.c_int, c_vp]),
    "tc_gemm_tile_plan": (ctypes.c_int, [c_i64, c_i64, c_i64, ctypes.c_int]),
    "tc_gemm_host_workspace_bytes": (c_i64, [c_i64, c_i64, c_i64]),
    "tc_gemm_f16_f32_host": (ctypes.c_int, [c_vp, c_vp, c_vp, c_i64, c_i64, c_i64, c_vp, c_i64, c_vp]),
    "tc_b2b_gemm_f16": (ctypes.c_int, [c_vp, c_vp, c_vp, c_vp, c_i64, c_i64, c_i64, c_i64, c_i64, c_vp]),
    "tc_flash_attn_fwd_f16": (
        ctypes.c_int,
        [c_vp, c_vp, c_vp, c_vp, c_vp, c_i64, c_i64, c_i64, c_i64, c_i64, c_i64, ctypes.c_float, ctypes.c_int, c_vp],
    ),
    "tc_flash_attn_fwd_ex_f16": (
        ctypes.c_int,
        [c_vp, c_vp, c_vp, c_vp, c_vp, c_i64, c_i64, c_i64, c_i64, c_i64, c_i64, ctypes.c_float, ctypes.c_int,
         ctypes.c_int, ctypes.c_int, c_vp],
    ),
    "tc_lstm_cell_f16": (ctypes.c_int, [c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_i64, c_i64, c_i64, c_vp]),
    "tc_lstm_chain_f16": (
        ctypes.c_int,
        [c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_i64, c_i64, c_i64, c_i64, c_vp],
    ),
    "tc_lstm_chain_workspace_bytes": (c_i64, [c_i64, c_i64, c_i64]),
    "tc_lstm_chain_ws_f16": (
        ctypes.c_int,
        [c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_i64, c_i64, c_i64, c_i64, c_vp, c_i64, c_vp],
    ),
    "tc_lstm_chain_static_f16": (
        ctypes.c_int,
        [c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_i64, c_i64, c_i64, c_i64, c_vp],
    ),
    "tc_peer_export": (ctypes.c_int, [c_vp, c_vp, c_i64]),
    "tc_peer_open": (ctypes.c_int, [c_vp, c_i64, ctypes.POINTER(c_vp)]),
    "tc_peer_close": (ctypes.c_int, [c_vp]),
    "tc_peer_copy": (ctypes.c_int, [c_vp, c_vp, c_i64, c_vp]),
    "tc_scatter_nd": (
        ctypes.c_int,
        [c_vp, c_vp, c_vp, ctypes.c_int, ctypes.POINTER(c_i64), ctypes.c_int, c_i64, ctypes.c_int, ctypes.c_int, c_vp],
    ),
    "tc_scatter_nd_add": (
        ctypes.c_int,
        [c_vp, c_vp, c_vp, ctypes.c_int, ctypes.POINTER(c_i64), ctypes.c_int, c_i64, ctypes.c_int, ctypes.c_int, c_vp],
    ),
}


class TiledCudaError(RuntimeError):
    """A C-ABI call returned a non-zero status."""

    def __init__(self, fn: str, status: int, message: str):
        super().__init__(f"{fn} failed with status {status}: {message}")
        self.status = status


_lib = None


def load() -> ctypes.CDLL:
    """Loads the native library once and declares every entry point."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m tiledcuda_b200.build` "
            "(there is no CPU or PyTorch fallback for these ops)"
        )
    lib = ctypes.CDLL(os.fspath(LIB_PATH))
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here means the build is stale
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def check(fn: str, status: int) -> None:
    if status != 0:
        msg = load().tc_last_error()
        raise TiledCudaError(fn, status, msg.decode("utf-8", "replace") if msg else "")


def device_status() -> int:
    """Reads and clears the device status word (synchronises the current device)."""
    code = ctypes.c_int(0)
    check("tc_device_status", load().tc_device_status(ctypes.byref(code)))
    return code.value
