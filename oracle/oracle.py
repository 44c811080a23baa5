"""CPU restatement of what the reference computes on the tile-kernel path. TEST INFRASTRUCTURE ONLY:
the checker for tests/, smoke() and the CPU-baseline legs of bench.py; never imported by the product.

Each function names the reference file:line whose computation it restates. Floating-point oracles
run in fp32 on the fp16-rounded inputs (the reference's own tests do the same with torch on the CPU);
scatter_nd is integer / byte work and is restated in numpy, bit-exact.

How this oracle is pinned:
  * flash_attention: against vectors produced by the reference's own Python oracle class
    (tests/python/test_flash_attn.py:9-75) imported from the reference tree, stored under
    tests/golden/, and against the reference's own host C++ oracle `host_flash_attn`
    (examples/cpp/03_flash_attention/flash_attn_cpu.hpp:9-100) compiled into oracle/_ref/.
  * scatter_nd: against vectors made with the reference test's own statement
    `data[indices[:, 0], indices[:, 1]] = updates` (tests/python/test_scatter_nd.py:46).
  * gemm: against the naive fp32 triple loop and the `i % 2048 / 1000` input ramp of
    tests/cpp/cell/test_single_wmma.cu:16-29, 58-62, restated in tests/golden/make_golden.py.
  * back2back_gemm: the reference checks it against two cuBLAS calls only (closed library, needs a
    GPU): examples/cpp/02_fused_two_gemms/util.hpp:29-119. Parity unpinned beyond that statement.
  * lstm_cell: the reference snapshot has no implementation and no test. Parity unpinned by the
    reference; the math is torch.nn.LSTMCell's, and the golden vectors come from torch.nn.LSTMCell.
"""
from __future__ import annotations

import math

import numpy as np
import torch

SEED = 1234  # the seed of the reference's Python tests (tests/python/test_flash_attn.py:81)


# --------------------------------------------------------------------------------------------------
# oracles
# --------------------------------------------------------------------------------------------------
def gemm(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """C = A @ B^T in fp32 from fp16 A [M,K] and B [N,K] (B is the column-major [K,N] operand).

    Reference: `a @ b.t()` (examples/python/gemm/main.py:21, 49-51); the naive fp32 loop
    `C[i][j] += A[i][k] * B[k + j*K]` (tests/cpp/cell/test_single_wmma.cu:16-29).
    """
    return a.detach().cpu().float() @ b.detach().cpu().float().t()


def gemm_naive(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """The triple loop itself, fp32 accumulate in k order (small cases only).

    Reference: tests/cpp/cell/test_single_wmma.cu:16-29.
    """
    a32 = a.astype(np.float32)
    b32 = b.astype(np.float32)
    m, k = a32.shape
    n = b32.shape[0]
    c = np.zeros((m, n), dtype=np.float32)
    for kk in range(k):
        c += np.outer(a32[:, kk], b32[:, kk]).astype(np.float32)
    return c


def back2back_gemm(a: torch.Tensor, b: torch.Tensor, d: torch.Tensor) -> torch.Tensor:
    """E = fp16(A @ B^T) @ D^T with fp32 accumulation; A [.., M,K], B [.., N,K], D [.., P,N].

    Reference: fp32 accumulator of the first product converted to fp16 in registers, then the second
    mma into an fp32 accumulator (examples/cpp/02_fused_two_gemms/fused_gemm.hpp:165-173); operand
    layouts A, output row-major, B and the second weight column-major (util.hpp:20-28, 52-63).
    """
    a32, b32, d32 = (t.detach().cpu().float() for t in (a, b, d))
    inter = (a32 @ b32.transpose(-1, -2)).half().float()
    return inter @ d32.transpose(-1, -2)


def flash_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float | None = None,
                    causal: bool = False):
    """(O, LSE) with O = softmax(scale * Q K^T) V in fp32 from fp16 Q [..,Sq,D], K [..,Skv,D], V [..,Skv,Dv].

    Reference: mathematically what the blockwise recurrences compute (tests/python/test_flash_attn.py:27-75;
    examples/cpp/03_flash_attention/flash_attn_cpu.hpp:9-100; src/kernels/flash_attn.cu:237-306). The
    reference applies no scale (scale = 1); the benchmark configuration uses 1/sqrt(D). causal (which the
    reference does not have) hides KV row j from query row i when j > i + (Skv - Sq); a row that sees
    nothing yields zeros and LSE = -inf.
    """
    q32, k32, v32 = (t.detach().cpu().float() for t in (q, k, v))
    if scale is None:
        scale = 1.0 / math.sqrt(q32.shape[-1])
    s = (q32 @ k32.transpose(-1, -2)) * scale
    if causal:
        sq, skv = s.shape[-2], s.shape[-1]
        i = torch.arange(sq).unsqueeze(1)
        j = torch.arange(skv).unsqueeze(0)
        s = s.masked_fill(j > i + (skv - sq), float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    prob = torch.exp(s - lse.unsqueeze(-1).clamp_min(-3.0e38))
    return prob @ v32, lse


def flash_attention_blockwise(q: torch.Tensor, k_t: torch.Tensor, v: torch.Tensor, block_n: int,
                              upcast: bool = False) -> torch.Tensor:
    """The reference's blockwise online-softmax recurrence, statement for statement.

    q [M,K]; k_t [K,N] (K already transposed, as the reference test passes it); v [N,P]; no scale.
    Reference: tests/python/test_flash_attn.py:27-75. With upcast=False the operands keep their dtype
    as they do in the reference, whose test feeds fp16 tensors, so products, exponentials and sums
    are rounded to fp16 while the running maxima, sums and output are fp32 (torch type promotion).
    With upcast=True everything is fp32. One deliberate difference: the running output starts at
    zero; the reference starts from torch.empty (:25) and multiplies it by prev_sums = 0 (:67), which
    yields NaN whenever the uninitialised buffer holds a non-finite value.
    """
    q, k_t, v = (t.detach().cpu() for t in (q, k_t, v))
    if upcast:
        q, k_t, v = q.float(), k_t.float(), v.float()
    m = q.shape[0]
    n = k_t.shape[1]
    out = torch.zeros(m, v.shape[1])
    prev_max = torch.zeros(m, 1)
    prev_sum = torch.zeros(m, 1)
    for n0 in range(0, n, block_n):
        kb = k_t[:, n0:n0 + block_n]
        vb = v[n0:n0 + block_n]
        w = q @ kb
        cur_max = w.max(dim=-1, keepdim=True).values
        e = torch.exp(w - cur_max)
        ev = e @ vb
        cur_sum = e.sum(dim=-1, keepdim=True)
        new_max = torch.maximum(cur_max, prev_max)
        renorm_prev = torch.exp(prev_max - new_max)
        renorm_cur = torch.exp(cur_max - new_max)
        new_sum = renorm_prev * prev_sum + renorm_cur * cur_sum
        out = (out * prev_sum * renorm_prev + renorm_cur * ev) / new_sum
        prev_sum, prev_max = new_sum, new_max
    return out


def lstm_cell(w, u, bias, x, h_prev, c_prev):
    """(h, c) of one LSTM cell in fp32, gate order (i, f, g, o) as torch.nn.LSTMCell.

    gates = x W^T + h U^T + b; c' = sigmoid(f) c + sigmoid(i) tanh(g); h' = sigmoid(o) tanh(c').
    The reference snapshot has no lstm_cell (only Makefile:3 names a test for it): parity unpinned.
    """
    w32, u32, x32, h32 = (t.detach().cpu().float() for t in (w, u, x, h_prev))
    c32 = c_prev.detach().cpu().float()
    gates = x32 @ w32.t() + h32 @ u32.t()
    if bias is not None:
        gates = gates + bias.detach().cpu().float()
    i, f, g, o = gates.chunk(4, dim=1)
    c = torch.sigmoid(f) * c32 + torch.sigmoid(i) * torch.tanh(g)
    h = torch.sigmoid(o) * torch.tanh(c)
    return h, c


def lstm_chain(w, u, bias, x, h0, c0):
    """(h_all [T,B,H], c_T): the cell applied over x [T,B,I]; c stays fp32, h is rounded to fp16 between steps."""
    h = h0.detach().cpu().float()
    c = c0.detach().cpu().float()
    hs = []
    for t in range(x.shape[0]):
        h, c = lstm_cell(w, u, bias, x[t], h.half(), c)
        hs.append(h)
    return torch.stack(hs), c


def scatter_nd(data: np.ndarray, indices: np.ndarray, updates: np.ndarray) -> np.ndarray:
    """ScatterND assignment on a copy of `data`: out[idx[t,0],...,idx[t,k-1]] = updates[t]. Bit-exact.

    Reference: the test's own oracle `data[indices[:, 0], indices[:, 1]] = updates`
    (tests/python/test_scatter_nd.py:46) and its update shape rule (:12-17). The reference kernel
    accumulates with atomicAdd instead (src/kernels/scatter_nd.cu:44-47) and never reads `updates`
    (:107); the assignment its test checks is what is restated here.
    """
    out = np.array(data, copy=True)
    k = indices.shape[-1]
    idx = indices.reshape(-1, k).astype(np.int64)
    upd = updates.reshape((idx.shape[0],) + out.shape[k:])
    out[tuple(idx[:, j] for j in range(k))] = upd
    return out


def scatter_nd_add(data: np.ndarray, indices: np.ndarray, updates: np.ndarray) -> np.ndarray:
    """ScatterND accumulation on a copy of `data`: out[idx[t,...]] += updates[t], repeated tuples adding up.

    Reference: the kernel's per-element atomicAdd (src/kernels/scatter_nd.cu:25-50, additions at :44-47).
    Sums run in tuple order (np.add.at); the device order is unspecified, so floating-point results with
    repeated tuples agree to rounding, integer results exactly.
    """
    out = np.array(data, copy=True)
    k = indices.shape[-1]
    idx = indices.reshape(-1, k).astype(np.int64)
    upd = updates.reshape((idx.shape[0],) + out.shape[k:])
    np.add.at(out, tuple(idx[:, j] for j in range(k)), upd)
    return out


def scatter_update_shape(index_dims, input_dims):
    """Shape of `updates` for given index and data shapes. Reference: tests/python/test_scatter_nd.py:12-17."""
    end = index_dims[-1]
    return list(index_dims[:-1]) + list(input_dims[end:])


# --------------------------------------------------------------------------------------------------
# seeded synthetic inputs with the shapes and value distributions of the benchmark configurations
# --------------------------------------------------------------------------------------------------
def _gen(seed: int) -> torch.Generator:
    return torch.Generator(device="cpu").manual_seed(seed)


def gemm_inputs(m: int, n: int, k: int, seed: int = SEED):
    """A [M,K] and B [N,K] fp16, entries uniform in [-1, 1)."""
    g = _gen(seed)
    a = (torch.rand(m, k, generator=g) * 2 - 1).half()
    b = (torch.rand(n, k, generator=g) * 2 - 1).half()
    return a, b


def b2b_inputs(m: int, n: int, k: int, p: int, batch: int = 1, seed: int = SEED):
    """A [b,M,K], B [b,N,K], D [b,P,N] fp16, entries normal(0, 0.1)."""
    g = _gen(seed)
    a = (torch.randn(batch, m, k, generator=g) * 0.1).half()
    b = (torch.randn(batch, n, k, generator=g) * 0.1).half()
    d = (torch.randn(batch, p, n, generator=g) * 0.1).half()
    return a, b, d


def attention_inputs(batch: int, heads: int, sq: int, skv: int, d: int, dv: int | None = None, seed: int = SEED):
    """Q [B,H,Sq,D], K [B,H,Skv,D], V [B,H,Skv,Dv] fp16, entries normal(0, 1)."""
    g = _gen(seed)
    dv = d if dv is None else dv
    q = torch.randn(batch, heads, sq, d, generator=g).half()
    k = torch.randn(batch, heads, skv, d, generator=g).half()
    v = torch.randn(batch, heads, skv, dv, generator=g).half()
    return q, k, v


def lstm_inputs(steps: int, batch: int, inp: int, hidden: int, seed: int = SEED, with_bias: bool = False):
    """W [4H,I], U [4H,H] fp16 normal(0, 0.02); x [T,B,I] fp16 normal(0,1); h0 = c0 = 0; bias zero or normal(0,0.1)."""
    g = _gen(seed)
    w = (torch.randn(4 * hidden, inp, generator=g) * 0.02).half()
    u = (torch.randn(4 * hidden, hidden, generator=g) * 0.02).half()
    x = torch.randn(steps, batch, inp, generator=g).half()
    h0 = torch.zeros(batch, hidden, dtype=torch.float16)
    c0 = torch.zeros(batch, hidden, dtype=torch.float32)
    bias = (torch.randn(4 * hidden, generator=g) * 0.1) if with_bias else None
    return w, u, bias, x, h0, c0


def scatter_inputs(rows: int, width: int, n: int, seed: int = SEED, index_dtype=torch.int32):
    """table [rows,width] fp16 normal; n unique row indices (first n of a seeded permutation); updates [n,width]."""
    g = _gen(seed)
    table = torch.randn(rows, width, generator=g).half()
    idx = torch.randperm(rows, generator=g)[:n].to(index_dtype).view(n, 1)
    upd = torch.randn(n, width, generator=g).half()
    return table, idx, upd


# --------------------------------------------------------------------------------------------------
# error metrics and the tolerances of the fp16-in / fp32-accumulate paths
# --------------------------------------------------------------------------------------------------
MAX_ABS_TOL = 2e-2
REL_FRO_TOL = 1e-3


def max_abs_err(out: torch.Tensor, ref: torch.Tensor) -> float:
    diff = (out.detach().cpu().float() - ref.detach().cpu().float()).abs()
    if torch.isnan(diff).any():
        return float("inf")
    return diff.max().item() if diff.numel() else 0.0


def rel_fro_err(out: torch.Tensor, ref: torch.Tensor) -> float:
    o = out.detach().cpu().float()
    r = ref.detach().cpu().float()
    if torch.isnan(o).any():
        return float("inf")
    denom = torch.linalg.norm(r).item()
    return torch.linalg.norm(o - r).item() / denom if denom > 0 else torch.linalg.norm(o - r).item()


def within_tolerance(out: torch.Tensor, ref: torch.Tensor, max_abs: float = MAX_ABS_TOL, rel_fro: float = REL_FRO_TOL) -> bool:
    return max_abs_err(out, ref) <= max_abs and rel_fro_err(out, ref) <= rel_fro
