"""Operators of the tile-kernel path on torch CUDA tensors, each a thin call into the C ABI.

Tensors supply device memory and the current stream; all arithmetic happens in the sm_100a kernels
of libtiledcuda_b200.so. Outputs are written in place into caller-allocated tensors, as the
reference's ops do (include/kernels/flash_attn.hpp:35-37, include/kernels/scatter_nd.hpp:39-40).
Nothing here falls back to PyTorch: a CPU tensor, a wrong dtype or an unsupported shape raises.
"""
from __future__ import annotations

import ctypes
import math

import torch

from . import _lib


import contextlib

_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_NO_GUARD = contextlib.nullcontext()


def _stream() -> ctypes.c_void_p:
    """The current CUDA stream of the current device as a raw handle."""
    if _raw_stream is not None:
        return ctypes.c_void_p(_raw_stream(torch.cuda.current_device()))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _on(device: torch.device):
    """Context that makes `device` current for the call; free when it already is (the usual case)."""
    if device.index is None or device.index == torch.cuda.current_device():
        return _NO_GUARD
    return torch.cuda.device(device)


def _ptr(t: torch.Tensor | None) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _need(t: torch.Tensor, name: str, dtype: torch.dtype, contiguous: bool = True) -> None:
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{name} must be a torch.Tensor")
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor (there is no CPU path)")
    if t.dtype != dtype:
        raise TypeError(f"{name} must be {dtype}, got {t.dtype}")
    if contiguous and not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")


def gemm(a: torch.Tensor, b: torch.Tensor, c: torch.Tensor, max_sms: int = 0) -> None:
    """c[M,N] (fp32) = a[M,K] @ b[N,K].T with fp16 (or bf16) inputs and fp32 accumulation.

    `b` is the column-major [K,N] operand of the reference's GEMM stored as [N,K] rows, so the result
    equals `a @ b.t()` (examples/python/gemm/main.py:21). Row strides of a, b, c may exceed the row
    length (leading dimensions); the innermost stride must be 1. max_sms > 0 (fp16 only) runs the GEMM on
    at most that many SMs and leaves the rest to kernels running beside it (tc_gemm_f16_f32_sms).
    """
    in_dtype = torch.bfloat16 if isinstance(a, torch.Tensor) and a.dtype == torch.bfloat16 else torch.float16
    for t, name, dt in ((a, "a", in_dtype), (b, "b", in_dtype), (c, "c", torch.float32)):
        _need(t, name, dt, contiguous=False)
        if t.dim() != 2 or t.stride(1) != 1:
            raise ValueError(f"{name} must be 2-D with unit inner stride")
    m, k = a.shape
    n, kb = b.shape
    if kb != k or tuple(c.shape) != (m, n):
        raise ValueError(f"shape mismatch: a {tuple(a.shape)}, b {tuple(b.shape)}, c {tuple(c.shape)}")
    lib = _lib.load()
    if max_sms:
        if in_dtype != torch.float16:
            raise ValueError("max_sms is supported for fp16 inputs only")
        with _on(a.device):
            _lib.check("tc_gemm_f16_f32_sms",
                       lib.tc_gemm_f16_f32_sms(_ptr(a), _ptr(b), _ptr(c), m, n, k, a.stride(0), b.stride(0), c.stride(0),
                                               int(max_sms), _stream()))
        return
    fn_name = "tc_gemm_bf16_f32" if in_dtype == torch.bfloat16 else "tc_gemm_f16_f32"
    with _on(a.device):
        _lib.check(
            fn_name,
            getattr(lib, fn_name)(_ptr(a), _ptr(b), _ptr(c), m, n, k, a.stride(0), b.stride(0), c.stride(0), _stream()),
        )


def gemm_host(a: torch.Tensor, b: torch.Tensor, c: torch.Tensor, workspace: torch.Tensor) -> None:
    """c (host, fp32 [M,N]) = a (host, fp16 [M,K]) @ b (host, fp16 [N,K]).T, copies pipelined against the kernel.

    a, b, c are contiguous CPU tensors (pinned for the copies to overlap); workspace is a CUDA uint8 tensor of
    at least gemm_host_workspace_bytes(M, N, K) bytes on the device that does the work. Everything is queued
    on return; synchronise the current stream of that device before reading c.
    """
    for t, name, dt in ((a, "a", torch.float16), (b, "b", torch.float16), (c, "c", torch.float32)):
        if t.is_cuda or t.dtype != dt or t.dim() != 2 or not t.is_contiguous():
            raise ValueError(f"{name} must be a contiguous 2-D CPU tensor of {dt}")
    if not workspace.is_cuda or not workspace.is_contiguous():
        raise ValueError("workspace must be a contiguous CUDA tensor")
    m, k = a.shape
    n, kb = b.shape
    if kb != k or tuple(c.shape) != (m, n):
        raise ValueError(f"shape mismatch: a {tuple(a.shape)}, b {tuple(b.shape)}, c {tuple(c.shape)}")
    lib = _lib.load()
    with _on(workspace.device):
        _lib.check(
            "tc_gemm_f16_f32_host",
            lib.tc_gemm_f16_f32_host(_ptr(a), _ptr(b), _ptr(c), m, n, k, _ptr(workspace),
                                     workspace.numel() * workspace.element_size(), _stream()),
        )


def gemm_host_workspace_bytes(m: int, n: int, k: int) -> int:
    return int(_lib.load().tc_gemm_host_workspace_bytes(m, n, k))


def back2back_gemm(a: torch.Tensor, b: torch.Tensor, d: torch.Tensor, e: torch.Tensor) -> None:
    """e (fp32 [.., M, P]) = fp16(a @ b.T) @ d.T, the intermediate kept on chip.

    a fp16 [batch, M, K] or [M, K]; b fp16 [.., N, K] (column-major [K,N]); d fp16 [.., P, N]
    (column-major [N,P]); as in KeFusedGemm (examples/cpp/02_fused_two_gemms/fused_gemm.hpp:98-181).
    """
    for t, name, dt in ((a, "a", torch.float16), (b, "b", torch.float16), (d, "d", torch.float16), (e, "e", torch.float32)):
        _need(t, name, dt)
    if a.dim() not in (2, 3) or b.dim() != a.dim() or d.dim() != a.dim() or e.dim() != a.dim():
        raise ValueError("a, b, d, e must all be 2-D or all be 3-D (batched)")
    batch = a.shape[0] if a.dim() == 3 else 1
    m, k = a.shape[-2:]
    n, kb = b.shape[-2:]
    p, nd = d.shape[-2:]
    if kb != k or nd != n or tuple(e.shape[-2:]) != (m, p):
        raise ValueError(f"shape mismatch: a {tuple(a.shape)}, b {tuple(b.shape)}, d {tuple(d.shape)}, e {tuple(e.shape)}")
    if a.dim() == 3 and not (b.shape[0] == d.shape[0] == e.shape[0] == batch):
        raise ValueError("batch sizes differ")
    lib = _lib.load()
    with _on(a.device):
        _lib.check("tc_b2b_gemm_f16", lib.tc_b2b_gemm_f16(_ptr(a), _ptr(b), _ptr(d), _ptr(e), m, n, k, p, batch, _stream()))


def flash_attn(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    o: torch.Tensor,
    scale: float | None = None,
    lse: torch.Tensor | None = None,
    v_is_transposed: bool = False,
    causal: bool = False,
    seq_major: bool = False,
) -> None:
    """o = softmax(scale * q k^T) v per (batch, head); fp32 statistics.

    q [B,H,Sq,D], k [B,H,Skv,D], o [B,H,Sq,Dv] fp16; v [B,H,Skv,Dv], or [B,H,Dv,Skv] when
    v_is_transposed. With seq_major the four tensors are [B,S,H,D] instead. scale defaults to
    1/sqrt(D). lse, if given, is fp32 [B,H,Sq]. causal: query row i sees KV rows
    j <= i + (Skv - Sq); a row that sees none comes back as zeros.
    """
    for t, name in ((q, "q"), (k, "k"), (v, "v"), (o, "o")):
        _need(t, name, torch.float16)
        if t.dim() != 4:
            raise ValueError(f"{name} must be 4-D [batch, heads, seq, dim]")
    if seq_major:
        if v_is_transposed:
            raise ValueError("a transposed v is not supported with seq_major operands")
        b, sq, h, d = q.shape
        skv = k.shape[1]
        dv = v.shape[3]
        k_expect, v_expect, o_expect = (b, skv, h, d), (b, skv, h, dv), (b, sq, h, dv)
    else:
        b, h, sq, d = q.shape
        skv = k.shape[2]
        dv = v.shape[2] if v_is_transposed else v.shape[3]
        k_expect = (b, h, skv, d)
        v_expect = (b, h, dv, skv) if v_is_transposed else (b, h, skv, dv)
        o_expect = (b, h, sq, dv)
    if tuple(k.shape) != k_expect or tuple(v.shape) != v_expect or tuple(o.shape) != o_expect:
        raise ValueError(f"shape mismatch: q {tuple(q.shape)}, k {tuple(k.shape)}, v {tuple(v.shape)}, o {tuple(o.shape)}")
    if lse is not None:
        _need(lse, "lse", torch.float32)
        if tuple(lse.shape) != (b, h, sq):
            raise ValueError("lse must be [batch, heads, seq_q]")
    if scale is None:
        scale = 1.0 / math.sqrt(d)
    lib = _lib.load()
    with _on(q.device):
        if causal or seq_major:
            _lib.check(
                "tc_flash_attn_fwd_ex_f16",
                lib.tc_flash_attn_fwd_ex_f16(
                    _ptr(q), _ptr(k), _ptr(v), _ptr(o), _ptr(lse), b, h, sq, skv, d, dv, float(scale),
                    int(bool(v_is_transposed)), int(bool(causal)), int(bool(seq_major)), _stream(),
                ),
            )
        else:
            _lib.check(
                "tc_flash_attn_fwd_f16",
                lib.tc_flash_attn_fwd_f16(
                    _ptr(q), _ptr(k), _ptr(v), _ptr(o), _ptr(lse), b, h, sq, skv, d, dv, float(scale),
                    int(bool(v_is_transposed)), _stream(),
                ),
            )


def flash_attention_fwd(Q: torch.Tensor, K: torch.Tensor, V: torch.Tensor, O: torch.Tensor, m: int, n: int, k: int, p: int) -> None:
    """The reference's op, argument for argument (src/kernels/flash_attn.cu:424-456).

    Flattened fp16 buffers: Q is [m,k] row-major, K is [n,k] row-major (K as [seq, dim]), V is V^T
    = [p,n] row-major, O is [m,p]; one head, no softmax scale. Any m, n and k, p <= 128 that the
    kernel covers are accepted, not only the reference's three hard-coded shapes.
    """
    for t, name, numel in ((Q, "Q", m * k), (K, "K", n * k), (V, "V", n * p), (O, "O", m * p)):
        _need(t, name, torch.float16)
        if t.numel() != numel:
            raise ValueError(f"{name} has {t.numel()} elements, expected {numel}")
    lib = _lib.load()
    with torch.cuda.device(Q.device):
        _lib.check(
            "tc_flash_attn_fwd_f16",
            lib.tc_flash_attn_fwd_f16(_ptr(Q), _ptr(K), _ptr(V), _ptr(O), _ptr(None), 1, 1, m, n, k, p, 1.0, 1, _stream()),
        )


def lstm_cell(
    w: torch.Tensor,
    u: torch.Tensor,
    bias: torch.Tensor | None,
    x: torch.Tensor,
    h_prev: torch.Tensor,
    c_prev: torch.Tensor,
    h_out: torch.Tensor,
    c_out: torch.Tensor,
) -> None:
    """One LSTM cell step with gate order (i, f, g, o) as torch.nn.LSTMCell.

    gates = x @ w.T + h_prev @ u.T + bias; c_out = sigmoid(f) * c_prev + sigmoid(i) * tanh(g);
    h_out = sigmoid(o) * tanh(c_out). w fp16 [4H, I]; u fp16 [4H, H]; bias fp32 [4H] or None; x fp16
    [B, I]; h fp16 [B, H]; c fp32 [B, H].
    """
    _need(w, "w", torch.float16)
    _need(u, "u", torch.float16)
    _need(x, "x", torch.float16)
    _need(h_prev, "h_prev", torch.float16)
    _need(h_out, "h_out", torch.float16)
    _need(c_prev, "c_prev", torch.float32)
    _need(c_out, "c_out", torch.float32)
    if bias is not None:
        _need(bias, "bias", torch.float32)
    batch, inp = x.shape
    hidden = u.shape[1]
    if tuple(w.shape) != (4 * hidden, inp) or tuple(u.shape) != (4 * hidden, hidden):
        raise ValueError(f"weight shapes {tuple(w.shape)}, {tuple(u.shape)} do not match input {inp}, hidden {hidden}")
    for t, name in ((h_prev, "h_prev"), (h_out, "h_out"), (c_prev, "c_prev"), (c_out, "c_out")):
        if tuple(t.shape) != (batch, hidden):
            raise ValueError(f"{name} must be [{batch}, {hidden}]")
    if bias is not None and bias.numel() != 4 * hidden:
        raise ValueError("bias must have 4*hidden elements")
    if h_out.data_ptr() == h_prev.data_ptr():
        raise ValueError("h_out must not alias h_prev")
    lib = _lib.load()
    with _on(x.device):
        _lib.check(
            "tc_lstm_cell_f16",
            lib.tc_lstm_cell_f16(_ptr(w), _ptr(u), _ptr(bias), _ptr(x), _ptr(h_prev), _ptr(c_prev), _ptr(h_out),
                                 _ptr(c_out), batch, inp, hidden, _stream()),
        )


def lstm_chain(
    w: torch.Tensor,
    u: torch.Tensor,
    bias: torch.Tensor | None,
    x: torch.Tensor,
    h0: torch.Tensor,
    c0: torch.Tensor,
    h_all: torch.Tensor,
    c_out: torch.Tensor,
    workspace: torch.Tensor | None = None,
) -> None:
    """`steps` chained cells: x fp16 [T, B, I]; h_all fp16 [T, B, H] gets every h_t; c_out fp32 [B, H] gets c_T.

    With `workspace` (a CUDA tensor of at least lstm_chain_workspace_bytes(T, B, H) bytes) the input
    projections of all steps are computed first as one GEMM and each step only runs h @ U.T.
    """
    _need(w, "w", torch.float16)
    _need(u, "u", torch.float16)
    _need(x, "x", torch.float16)
    _need(h0, "h0", torch.float16)
    _need(h_all, "h_all", torch.float16)
    _need(c0, "c0", torch.float32)
    _need(c_out, "c_out", torch.float32)
    if bias is not None:
        _need(bias, "bias", torch.float32)
    steps, batch, inp = x.shape
    hidden = u.shape[1]
    if tuple(w.shape) != (4 * hidden, inp) or tuple(u.shape) != (4 * hidden, hidden):
        raise ValueError("weight shapes do not match x / hidden size")
    if tuple(h_all.shape) != (steps, batch, hidden) or tuple(h0.shape) != (batch, hidden):
        raise ValueError("h_all must be [steps, batch, hidden] and h0 [batch, hidden]")
    if tuple(c0.shape) != (batch, hidden) or tuple(c_out.shape) != (batch, hidden):
        raise ValueError("c0 and c_out must be [batch, hidden]")
    lib = _lib.load()
    with _on(x.device):
        if workspace is None:
            _lib.check(
                "tc_lstm_chain_f16",
                lib.tc_lstm_chain_f16(_ptr(w), _ptr(u), _ptr(bias), _ptr(x), _ptr(h0), _ptr(c0), _ptr(h_all), _ptr(c_out),
                                      steps, batch, inp, hidden, _stream()),
            )
        else:
            if not workspace.is_cuda or not workspace.is_contiguous():
                raise ValueError("workspace must be a contiguous CUDA tensor")
            _lib.check(
                "tc_lstm_chain_ws_f16",
                lib.tc_lstm_chain_ws_f16(_ptr(w), _ptr(u), _ptr(bias), _ptr(x), _ptr(h0), _ptr(c0), _ptr(h_all), _ptr(c_out),
                                         steps, batch, inp, hidden, _ptr(workspace), workspace.numel() * workspace.element_size(),
                                         _stream()),
            )


def lstm_chain_workspace_bytes(steps: int, batch: int, hidden: int) -> int:
    """Bytes of scratch memory lstm_chain needs to hoist the input projections out of the recurrence."""
    return int(_lib.load().tc_lstm_chain_workspace_bytes(steps, batch, hidden))


_SCATTER_ADD_TYPES = {torch.float32: 0, torch.float16: 1, torch.int32: 2, torch.float64: 3}


def _scatter_args(data: torch.Tensor, indices: torch.Tensor, updates: torch.Tensor):
    if not data.is_cuda or not indices.is_cuda or not updates.is_cuda:
        raise ValueError("scatter_nd needs CUDA tensors (there is no CPU path)")
    if indices.dtype not in (torch.int32, torch.int64):
        raise TypeError(f"indices must be int32 or int64, got {indices.dtype}")
    if updates.dtype != data.dtype:
        raise TypeError("updates and data must have the same dtype")
    if not (data.is_contiguous() and indices.is_contiguous() and updates.is_contiguous()):
        raise ValueError("data, indices and updates must be contiguous")
    if indices.dim() < 1:
        raise ValueError("indices must have at least one dimension")
    k = indices.shape[-1]
    n = indices.numel() // k if k else 0
    if k < 1 or k > data.dim():
        raise ValueError(f"index tuple length {k} does not fit data of rank {data.dim()}")
    slice_elems = 1
    for s in data.shape[k:]:
        slice_elems *= s
    if updates.numel() != n * slice_elems:
        raise ValueError(f"updates has {updates.numel()} elements, expected {n} slices of {slice_elems}")
    dims = (ctypes.c_int64 * data.dim())(*data.shape)
    return dims, n, k


def scatter_nd(data: torch.Tensor, indices: torch.Tensor, updates: torch.Tensor) -> None:
    """data[indices[t, 0], ..., indices[t, k-1]] = updates[t] for every index tuple t (in place).

    data is N-D and contiguous; indices is int32 or int64 [..., k]; updates holds one slice
    data.shape[k:] per tuple. Tuples must be unique for a deterministic result. Argument order follows
    the reference's Python wrapper (pytiledcuda/__init__.py:6-8): data, indices, updates.
    """
    dims, n, k = _scatter_args(data, indices, updates)
    lib = _lib.load()
    with _on(data.device):
        _lib.check(
            "tc_scatter_nd",
            lib.tc_scatter_nd(_ptr(data), _ptr(updates), _ptr(indices), int(indices.dtype == torch.int64), dims,
                              data.dim(), n, k, data.element_size(), _stream()),
        )


def scatter_nd_add(data: torch.Tensor, indices: torch.Tensor, updates: torch.Tensor) -> None:
    """data[indices[t, 0], ..., indices[t, k-1]] += updates[t] (in place); repeated tuples add up.

    What the reference's kernel does with one atomicAdd per element (src/kernels/scatter_nd.cu:44-47).
    fp32, fp16, int32 and fp64 tables; arguments as scatter_nd.
    """
    if data.dtype not in _SCATTER_ADD_TYPES:
        raise TypeError(f"scatter_nd_add supports {sorted(str(t) for t in _SCATTER_ADD_TYPES)}, got {data.dtype}")
    dims, n, k = _scatter_args(data, indices, updates)
    lib = _lib.load()
    with _on(data.device):
        _lib.check(
            "tc_scatter_nd_add",
            lib.tc_scatter_nd_add(_ptr(data), _ptr(updates), _ptr(indices), int(indices.dtype == torch.int64), dims,
                                  data.dim(), n, k, _SCATTER_ADD_TYPES[data.dtype], _stream()),
        )
