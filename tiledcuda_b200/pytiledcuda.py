"""The reference's Python surface (pytiledcuda/__init__.py:3-36) over torch.ops.tiledcuda.*.

Same names, argument orders and in-place conventions: scatter_nd(data, indices, updates),
flash_attention_fwd(Q, K, V, O, m, n, k, p) and class TiledFlashAttention(query, key, value), plus
the ops the reference only has as C++ examples (gemm, back2back_gemm) or only names (lstm_cell).
The op library is found beside this file, not relative to the working directory. Two differences
from the reference, both forced by what its kernel ignores: scatter_nd needs `data` and `indices`
with their real shapes (the reference's launcher cannot recover them from flattened tensors), and
scatter_nd really reads `updates` (the reference's launch passes the index buffer in its place,
src/kernels/scatter_nd.cu:107).
"""
from __future__ import annotations

import math
import os
from pathlib import Path

import torch

_OP_LIB = Path(__file__).resolve().parent / "libtiledcuda.so"
if not _OP_LIB.exists():
    raise ImportError(f"{_OP_LIB} is missing: build it with `python -m tiledcuda_b200.build --torch`")
torch.ops.load_library(os.fspath(_OP_LIB))


def scatter_nd(scatter_data, scatter_indices, scatter_updates):
    torch.ops.tiledcuda.scatter_nd(scatter_data, scatter_updates, scatter_indices)


def flash_attention_fwd(Q, K, V, O, m, n, k, p):
    torch.ops.tiledcuda.flash_attention_fwd(Q, K, V, O, m, n, k, p)


def flash_attn(Q, K, V, O, scale=None, v_is_transposed=False):
    if scale is None:
        scale = Q.shape[-1] ** -0.5
    torch.ops.tiledcuda.flash_attn(Q, K, V, O, float(scale), bool(v_is_transposed))


def flash_attn_ex(Q, K, V, O, scale=None, causal=False, seq_major=False):
    """flash_attn with a bottom-right aligned causal mask and / or [B, S, H, D] operands."""
    if scale is None:
        scale = 1.0 / math.sqrt(Q.shape[-1])
    torch.ops.tiledcuda.flash_attn_ex(Q, K, V, O, float(scale), bool(causal), bool(seq_major))


def scatter_nd_add(scatter_data, scatter_indices, scatter_updates):
    """Accumulating scatter, what the reference's kernel does (src/kernels/scatter_nd.cu:44-47); argument order as
    scatter_nd."""
    torch.ops.tiledcuda.scatter_nd_add(scatter_data, scatter_updates, scatter_indices)


def gemm(A, B, C):
    torch.ops.tiledcuda.gemm(A, B, C)


def back2back_gemm(A, B, D, E):
    torch.ops.tiledcuda.back2back_gemm(A, B, D, E)


def lstm_cell(W, U, bias, x, h_prev, c_prev, h_out, c_out):
    torch.ops.tiledcuda.lstm_cell(W, U, bias, x, h_prev, c_prev, h_out, c_out)


class TiledFlashAttention:
    """query [m,k], key [k,n] (already K^T, as the reference test passes it), value [n,p]; one head, no scale."""

    def __init__(self, query, key, value):
        self.m, self.k = query.size(-2), query.size(-1)
        self.n, self.p = value.size(-2), value.size(-1)
        self.query = query.half().flatten()
        self.key = key.half().t().flatten()      # [n, k] rows: K as [seq, dim]
        self.value = value.half().t().flatten()  # V^T = [p, n] rows
        self.output = torch.empty(self.m, self.p, dtype=torch.half, device=query.device).flatten()

    def forward(self) -> torch.Tensor:
        flash_attention_fwd(self.query, self.key, self.value, self.output, self.m, self.n, self.k, self.p)
        return self.output.view(self.m, self.p)
