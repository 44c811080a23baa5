"""CPU tests: the oracle against the golden vectors taken from the reference's own tests, and against
the reference's host C++ oracle when it has been built into oracle/_ref/."""
import ctypes
import math
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import oracle

REF_SO = Path(__file__).resolve().parent.parent / "oracle" / "_ref" / "libref_host_flash_attn.so"


@pytest.mark.parametrize("n", [64, 128, 256])
def test_flash_attention_matches_reference_python_oracle(golden_dir, n):
    g = np.load(golden_dir / f"flash_attn_ref_n{n}.npz")
    q, k_t, v, o_ref = (torch.from_numpy(g[x]) for x in ("q", "k_t", "v", "o"))
    m, nn, k, p, ktm, ktn, ktk, ktp = g["shape"].tolist()
    assert nn == n
    # statement-for-statement restatement on the same fp16 operands and block size: identical arithmetic
    blockwise = oracle.flash_attention_blockwise(q, k_t, v, ktn)
    assert oracle.max_abs_err(blockwise.half(), o_ref) <= 1e-6
    # the same recurrence in fp32, and the closed form the product is checked against (scale = 1, as in
    # the reference): they differ from the fp16-operand reference only by its fp16 rounding
    fp32_blockwise = oracle.flash_attention_blockwise(q, k_t, v, ktn, upcast=True)
    direct, _ = oracle.flash_attention(q, k_t.t(), v, scale=1.0)
    assert oracle.max_abs_err(fp32_blockwise, direct) <= 1e-5
    assert oracle.max_abs_err(direct, o_ref) <= 2e-2  # the reference test itself accepts 8e-2 (:114)
    # the tolerance of the reference's own test is 8e-2 per element (tests/python/test_flash_attn.py:114)


@pytest.mark.skipif(not REF_SO.exists(), reason="oracle/_ref not built (needs the reference checkout)")
@pytest.mark.parametrize("n", [64, 128, 256])
def test_flash_attention_matches_reference_host_cpp_oracle(golden_dir, n):
    """host_flash_attn works in fp16 throughout; its own example accepts 1e-1 per element."""
    g = np.load(golden_dir / f"flash_attn_ref_n{n}.npz")
    q, k_t, v = (torch.from_numpy(g[x]) for x in ("q", "k_t", "v"))
    m, k = q.shape
    p = v.shape[1]
    lib = ctypes.CDLL(str(REF_SO))
    k_rows = k_t.t().contiguous()  # [n, k]: K[j, kk] at kk + k*j
    v_t = v.t().contiguous()       # [p, n]: V[kk, j] at kk + n*j
    out = torch.zeros(m, p, dtype=torch.float16)
    lib.ref_host_flash_attn(m, n, k, p, ctypes.c_void_p(q.data_ptr()), ctypes.c_void_p(k_rows.data_ptr()),
                            ctypes.c_void_p(v_t.data_ptr()), ctypes.c_void_p(out.data_ptr()))
    direct, _ = oracle.flash_attention(q, k_rows, v, scale=1.0)
    # fp16 accumulation over k and n: the reference's example accepts 1e-1 per element against its kernel
    # (examples/cpp/03_flash_attention/util.hpp:16-30); the mean error shows there is no systematic difference
    assert oracle.max_abs_err(direct, out) <= 1.5e-1
    assert (direct - out.float()).abs().mean().item() <= 1e-2


def test_scatter_nd_matches_reference_test_statement(golden_dir):
    g = np.load(golden_dir / "scatter_nd_ref.npz")
    out = oracle.scatter_nd(g["data"], g["indices"], g["updates"])
    assert out.tobytes() == g["out"].tobytes()
    out2 = oracle.scatter_nd(g["data2"], g["indices2"], g["updates2"])
    assert out2.tobytes() == g["out2"].tobytes()
    assert oracle.scatter_update_shape([5, 2], [7, 8, 9, 10]) == [5, 9, 10]


def test_scatter_nd_edge_cases():
    data = np.arange(24, dtype=np.float32).reshape(4, 6)
    same = oracle.scatter_nd(data, np.zeros((0, 1), dtype=np.int64), np.zeros((0, 6), dtype=np.float32))
    assert same.tobytes() == data.tobytes()
    full = oracle.scatter_nd(data, np.array([[3], [0]]), np.ones((2, 6), dtype=np.float32))
    assert (full[3] == 1).all() and (full[0] == 1).all() and (full[1] == data[1]).all()
    elem = oracle.scatter_nd(data, np.array([[1, 2]]), np.array([99.0], dtype=np.float32))
    assert elem[1, 2] == 99.0 and elem.sum() == data.sum() - data[1, 2] + 99.0


@pytest.mark.parametrize("tag", ["16", "64x128x128"])
def test_gemm_matches_naive_ramp(golden_dir, tag):
    g = np.load(golden_dir / "gemm_ramp.npz")
    a, b, c = g[f"a_{tag}"], g[f"b_{tag}"], g[f"c_{tag}"]
    out = oracle.gemm(torch.from_numpy(a), torch.from_numpy(b))
    # the reference's device check is |a - b| < 1e-3 on this ramp (tests/cpp/cell/test_single_wmma.cu:32)
    assert np.abs(out.numpy() - c).max() < 1e-3
    assert np.abs(oracle.gemm_naive(a, b) - c).max() < 1e-3


def test_b2b_rounds_intermediate_to_fp16():
    a, b, d = oracle.b2b_inputs(64, 96, 32, 48, batch=2)
    e = oracle.back2back_gemm(a, b, d)
    unrounded = (a.float() @ b.float().transpose(1, 2)) @ d.float().transpose(1, 2)
    assert e.shape == (2, 64, 48)
    assert not torch.equal(e, unrounded)
    assert torch.allclose(e, unrounded, atol=1e-3)


def test_lstm_matches_torch_cell(golden_dir):
    g = np.load(golden_dir / "lstm_cell_torch.npz")
    t = {k: torch.from_numpy(g[k]) for k in g.files}
    h1, c1 = oracle.lstm_cell(t["w"], t["u"], t["bias"], t["x"], t["h"], t["c"])
    assert torch.allclose(h1, t["h1"], atol=1e-5) and torch.allclose(c1, t["c1"], atol=1e-5)


def test_lstm_chain_is_repeated_cell():
    w, u, bias, x, h0, c0 = oracle.lstm_inputs(3, 4, 16, 16, with_bias=True)
    hs, c = oracle.lstm_chain(w, u, bias, x, h0, c0)
    h, cc = h0.float(), c0
    for t in range(3):
        h, cc = oracle.lstm_cell(w, u, bias, x[t], h.half(), cc)
        assert torch.equal(hs[t], h)
    assert torch.equal(c, cc)


def test_input_generators_follow_the_configurations():
    a, b = oracle.gemm_inputs(32, 16, 64)
    assert a.dtype == torch.float16 and a.min() >= -1 and a.max() < 1 and b.shape == (16, 64)
    q, k, v = oracle.attention_inputs(1, 2, 8, 16, 32)
    assert q.shape == (1, 2, 8, 32) and k.shape == (1, 2, 16, 32) and v.shape == (1, 2, 16, 32)
    table, idx, upd = oracle.scatter_inputs(256, 8, 64)
    assert idx.dtype == torch.int32 and idx.unique().numel() == 64 and upd.shape == (64, 8)
    a2, _ = oracle.gemm_inputs(32, 16, 64)
    assert torch.equal(a, a2)
    assert math.isclose(oracle.rel_fro_err(a, a), 0.0)


def test_oracle_causal_attention_matches_torch_sdpa():
    """The causal option of the oracle against torch's scaled_dot_product_attention with an explicit mask."""
    for sq, skv in ((64, 64), (40, 100), (100, 40)):
        q, k, v = oracle.attention_inputs(1, 2, sq, skv, 32, 32)
        o, lse = oracle.flash_attention(q, k, v, causal=True)
        i = torch.arange(sq).unsqueeze(1)
        j = torch.arange(skv).unsqueeze(0)
        mask = j <= i + (skv - sq)
        want = torch.nn.functional.scaled_dot_product_attention(q.float(), k.float(), v.float(), attn_mask=mask)
        seen = mask.any(dim=1)
        assert torch.allclose(o[:, :, seen], want[:, :, seen], atol=1e-5)
        assert (o[:, :, ~seen] == 0).all() and torch.isinf(lse[:, :, ~seen]).all()


def test_oracle_scatter_nd_add_matches_loop_and_torch():
    """np.add.at restatement against a plain loop and torch.index_put_(accumulate=True)."""
    rng = np.random.default_rng(oracle.SEED)
    data = rng.integers(-5, 5, (6, 7, 3)).astype(np.float32)
    idx = rng.integers(0, (6, 7), (40, 2)).astype(np.int64)
    upd = rng.integers(-5, 5, (40, 3)).astype(np.float32)
    got = oracle.scatter_nd_add(data, idx, upd)
    want = data.copy()
    for t in range(40):
        want[idx[t, 0], idx[t, 1]] += upd[t]
    assert got.tobytes() == want.tobytes()
    tt = torch.from_numpy(data.copy())
    tt.index_put_((torch.from_numpy(idx[:, 0]), torch.from_numpy(idx[:, 1])), torch.from_numpy(upd), accumulate=True)
    assert tt.numpy().tobytes() == want.tobytes()
