"""GPU tests of the reference-facing Python surface (torch.ops.tiledcuda.* through tiledcuda_b200.pytiledcuda),
written the way the reference's own Python tests call it (tests/python/test_flash_attn.py:101-102,
tests/python/test_scatter_nd.py:43)."""
import numpy as np
import pytest
import torch

from oracle import oracle

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def ptc():
    assert torch.cuda.is_available()
    from tiledcuda_b200 import pytiledcuda

    return pytiledcuda


@pytest.mark.parametrize("n", [64, 128, 256])
def test_tiled_flash_attention_class(ptc, golden_dir, n):
    g = np.load(golden_dir / f"flash_attn_ref_n{n}.npz")
    q, k_t, v, o_ref = (torch.from_numpy(g[x]) for x in ("q", "k_t", "v", "o"))
    out = ptc.TiledFlashAttention(q.to(DEV), k_t.to(DEV), v.to(DEV)).forward()
    assert out.shape == o_ref.shape
    assert oracle.max_abs_err(out, o_ref) <= 2e-2  # the reference's test accepts 8e-2 per element


def test_scatter_nd_reference_call(ptc, golden_dir):
    g = np.load(golden_dir / "scatter_nd_ref.npz")
    data = torch.from_numpy(g["data"]).to(DEV)
    ptc.scatter_nd(data, torch.from_numpy(g["indices"]).to(DEV), torch.from_numpy(g["updates"]).to(DEV))
    assert data.cpu().numpy().tobytes() == g["out"].tobytes()
    # a flat view of the same storage sees the update, as the reference test expects of its in-place op
    assert torch.equal(data.flatten().cpu(), torch.from_numpy(g["out"]).flatten())


def test_new_ops_are_registered_and_match(ptc):
    a, b = oracle.gemm_inputs(256, 384, 128)
    c = torch.empty(256, 384, device=DEV)
    ptc.gemm(a.to(DEV), b.to(DEV), c)
    assert oracle.within_tolerance(c, oracle.gemm(a, b), 2e-3, 1e-5)

    a2, b2, d2 = oracle.b2b_inputs(256, 256, 128, 128, batch=2)
    e = torch.empty(2, 256, 128, device=DEV)
    ptc.back2back_gemm(a2.to(DEV), b2.to(DEV), d2.to(DEV), e)
    assert oracle.within_tolerance(e, oracle.back2back_gemm(a2, b2, d2))

    q, k, v = oracle.attention_inputs(1, 2, 128, 256, 64)
    o = torch.empty(1, 2, 128, 64, dtype=torch.float16, device=DEV)
    ptc.flash_attn(q.to(DEV), k.to(DEV), v.to(DEV), o)
    assert oracle.within_tolerance(o, oracle.flash_attention(q, k, v)[0])

    w, u, bias, x, h0, c0 = oracle.lstm_inputs(1, 64, 64, 32, with_bias=True)
    h1 = torch.empty(64, 32, dtype=torch.float16, device=DEV)
    c1 = torch.empty(64, 32, device=DEV)
    ptc.lstm_cell(w.to(DEV), u.to(DEV), bias.to(DEV), x[0].to(DEV), h0.to(DEV), c0.to(DEV), h1, c1)
    rh, rc = oracle.lstm_cell(w, u, bias, x[0], h0, c0)
    assert oracle.within_tolerance(h1, rh) and oracle.within_tolerance(c1, rc)
    ptc.lstm_cell(w.to(DEV), u.to(DEV), None, x[0].to(DEV), h0.to(DEV), c0.to(DEV), h1, c1)


def test_extended_ops_through_the_dispatcher(ptc):
    """Causal and sequence-major attention and the accumulating scatter as torch ops."""
    q, k, v = oracle.attention_inputs(1, 2, 256, 256, 64)
    o = torch.empty(1, 2, 256, 64, dtype=torch.float16, device=DEV)
    ptc.flash_attn_ex(q.to(DEV), k.to(DEV), v.to(DEV), o, causal=True)
    assert oracle.within_tolerance(o, oracle.flash_attention(q, k, v, causal=True)[0])
    to_sm = lambda t: t.to(DEV).transpose(1, 2).contiguous()
    o2 = torch.empty(1, 256, 2, 64, dtype=torch.float16, device=DEV)
    ptc.flash_attn_ex(to_sm(q), to_sm(k), to_sm(v), o2, causal=True, seq_major=True)
    assert torch.equal(o2.transpose(1, 2), o)

    g = torch.Generator().manual_seed(5)
    table = torch.randint(-8, 8, (300, 4), generator=g).float()
    idx = torch.randint(0, 300, (1000, 1), generator=g)
    upd = torch.randint(-4, 4, (1000, 4), generator=g).float()
    dev = table.to(DEV)
    ptc.scatter_nd_add(dev, idx.to(DEV), upd.to(DEV))
    assert dev.cpu().numpy().tobytes() == oracle.scatter_nd_add(table.numpy(), idx.numpy(), upd.numpy()).tobytes()


def test_errors_surface_as_runtime_errors(ptc):
    a = torch.zeros(128, 60, dtype=torch.float16, device=DEV)
    with pytest.raises(RuntimeError, match="multiple of 8"):
        ptc.gemm(a, a, torch.zeros(128, 128, device=DEV))
    with pytest.raises((RuntimeError, NotImplementedError)):
        ptc.gemm(a.cpu(), a.cpu(), torch.zeros(128, 128))  # no CPU kernel is registered


def test_reference_import_lines_work_unchanged():
    """`from pytiledcuda import TiledFlashAttention` (tests/python/test_flash_attn.py:6 of the reference) and
    `pytiledcuda.scatter_nd(data, indices, updates)` (tests/python/test_scatter_nd.py:43) import and run as written."""
    import pytiledcuda
    from pytiledcuda import TiledFlashAttention

    g = torch.Generator().manual_seed(1234)                     # the reference test's seed and shapes
    q = torch.randn(64, 128, generator=g).half().to(DEV)
    k_t = torch.randn(128, 128, generator=g).half().to(DEV)
    v = torch.randn(128, 128, generator=g).half().to(DEV)
    out = TiledFlashAttention(q, k_t, v).forward()
    ref, _ = oracle.flash_attention(q.cpu(), k_t.cpu().t().contiguous(), v.cpu(), scale=1.0)
    assert oracle.max_abs_err(out, ref) <= 2e-2

    data = torch.zeros(7, 8, 9, 10, device=DEV)
    idx = torch.tensor([[0, 1], [6, 7], [3, 3]], dtype=torch.int64, device=DEV)
    upd = torch.arange(3 * 90, dtype=torch.float32, device=DEV).view(3, 9, 10)
    pytiledcuda.scatter_nd(data, idx, upd)
    want = torch.zeros(7, 8, 9, 10)
    want[idx[:, 0].cpu(), idx[:, 1].cpu()] = upd.cpu()
    assert torch.equal(data.cpu(), want)


def test_wrong_shapes_raise_before_any_launch(ptc, clean_status):
    """The dispatcher-level ops refuse tensors whose shapes would send a kernel outside its buffers: each call below
    raises a RuntimeError from the argument checks, nothing is launched, and the device status word stays clean."""
    f16 = dict(dtype=torch.float16, device=DEV)
    table = torch.zeros(64, 8, **f16)
    idx = torch.zeros(10, 1, dtype=torch.int64, device=DEV)
    with pytest.raises(RuntimeError, match="updates has"):
        ptc.scatter_nd(table, idx, torch.zeros(9, 8, **f16))          # one slice short
    with pytest.raises(RuntimeError, match="updates has"):
        ptc.scatter_nd_add(table.float(), idx, torch.zeros(10, 4, device=DEV))
    with pytest.raises(RuntimeError, match="do not fit"):
        ptc.scatter_nd(table, torch.zeros(10, 3, dtype=torch.int64, device=DEV), torch.zeros(10, **f16))

    hidden, inp, batch = 32, 64, 64
    w, u = torch.zeros(4 * hidden, inp, **f16), torch.zeros(4 * hidden, hidden, **f16)
    x, h = torch.zeros(batch, inp, **f16), torch.zeros(batch, hidden, **f16)
    c = torch.zeros(batch, hidden, device=DEV)
    h_out, c_out = torch.empty_like(h), torch.empty_like(c)
    with pytest.raises(RuntimeError, match="must be"):
        ptc.lstm_cell(w, u, None, x, h[: batch // 2], c, h_out, c_out)           # h_prev too short
    with pytest.raises(RuntimeError, match="must be"):
        ptc.lstm_cell(w, u, None, x, h, c, h_out, c_out[:, : hidden // 2].contiguous())
    with pytest.raises(RuntimeError, match="bias must have"):
        ptc.lstm_cell(w, u, torch.zeros(hidden, device=DEV), x, h, c, h_out, c_out)
    with pytest.raises(RuntimeError, match="alias"):
        ptc.lstm_cell(w, u, None, x, h, c, h, c_out)
    with pytest.raises(RuntimeError, match="2-D"):
        ptc.lstm_cell(w, u, None, x.view(1, batch, inp), h, c, h_out, c_out)
    with pytest.raises(RuntimeError, match="weight shape"):
        ptc.lstm_cell(w, torch.zeros(4 * hidden, hidden + 16, **f16), None, x, h, c, h_out, c_out)

    if torch.cuda.device_count() > 1:
        a = torch.zeros(128, 64, **f16)
        with pytest.raises(RuntimeError, match="one device"):
            ptc.gemm(a, a.to("cuda:1"), torch.zeros(128, 128, device=DEV))
