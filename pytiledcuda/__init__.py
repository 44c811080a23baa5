"""`pytiledcuda`, under the reference's own package name.

The reference's tests and examples write `from pytiledcuda import TiledFlashAttention`
(tests/python/test_flash_attn.py:6) and `import pytiledcuda` (tests/python/test_scatter_nd.py:3,
examples/python/scatter_nd.py); with this directory on the path they import unchanged. Everything
is defined in tiledcuda_b200.pytiledcuda, which loads the op library that lies beside it (not a path
relative to the working directory, as pytiledcuda/__init__.py:3 of the reference does).
"""
from tiledcuda_b200.pytiledcuda import (  # noqa: F401
    TiledFlashAttention,
    back2back_gemm,
    flash_attention_fwd,
    flash_attn,
    flash_attn_ex,
    gemm,
    lstm_cell,
    scatter_nd,
    scatter_nd_add,
)

__all__ = [
    "TiledFlashAttention",
    "back2back_gemm",
    "flash_attention_fwd",
    "flash_attn",
    "flash_attn_ex",
    "gemm",
    "lstm_cell",
    "scatter_nd",
    "scatter_nd_add",
]
