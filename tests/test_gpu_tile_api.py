"""GPU tests of the C++ tile API (tiledcuda_b200/include): kernels written with GlobalTile / SharedTile /
TmemTile / RegTile, the tile iterators, the loaders and storers, compute::gemm and the register-tile
operations, compiled into tests/cpp/libtile_api_tests.so. The cases replay the shapes of the reference's
single-CTA unit tests (tests/cpp/cell/test_gemm.cu:306-351, test_g2s_load.cu:118-144,
test_swizzled_copy.cu:399-499, test_softmax.cu:117-163); results are compared on the host with the CPU oracle."""
import ctypes
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import oracle

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
LIB = Path(__file__).resolve().parent / "cpp" / "libtile_api_tests.so"


@pytest.fixture(scope="module")
def lib():
    assert torch.cuda.is_available()
    assert LIB.exists(), f"{LIB} is missing: build it with `python -m tiledcuda_b200.build --tests`"
    torch.cuda.set_device(0)
    return ctypes.CDLL(str(LIB))


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


def test_case_counts(lib):
    assert lib.tcx_gemm_case_count() == 43 and lib.tcx_roundtrip_case_count() == 42


@pytest.mark.parametrize("case", range(42))
def test_global_shared_round_trip_is_exact(lib, case):
    """global -> shared (swizzled / interleaved operand layout, or plain fp32) -> global reproduces the data."""
    src = torch.empty(128 * 256, dtype=torch.float32, device=DEV)
    dst = torch.full((128 * 256,), -1.0, dtype=torch.float32, device=DEV)
    rows, cols, elem, cm = (ctypes.c_int() for _ in range(4))
    # first call only to learn the shape (output is discarded), then the real call on a ramp
    assert lib.tcx_roundtrip(case, _p(src), _p(dst), ctypes.byref(rows), ctypes.byref(cols), ctypes.byref(elem), ctypes.byref(cm)) == 0
    torch.cuda.synchronize()
    n = rows.value * cols.value
    dtype = torch.float16 if elem.value == 2 else torch.float32
    ramp = (torch.arange(n, device=DEV) % 2048).to(dtype)   # the `i % 2048` ramp of test_g2s_load.cu:39-40
    out = torch.full((n,), -1, dtype=dtype, device=DEV)
    assert lib.tcx_roundtrip(case, _p(ramp), _p(out), ctypes.byref(rows), ctypes.byref(cols), ctypes.byref(elem), ctypes.byref(cm)) == 0
    torch.cuda.synchronize()
    assert torch.equal(out, ramp)


@pytest.mark.parametrize("swizzled", [1, 0])
@pytest.mark.parametrize("case", range(37))
def test_chunked_round_trip_reference_shapes(lib, case, swizzled):
    """The 24 row-major and 13 column-major shapes of the reference's swizzled-load tests
    (tests/cpp/cell/test_swizzled_copy.cu:399-449), walked chunk by chunk with a GTileIterator through a shared
    operand tile in both operand layouts; the output must reproduce the `i % 2048` ramp exactly."""
    assert lib.tcx_chunked_roundtrip_case_count() == 37
    rows, cols, cm = (ctypes.c_int() for _ in range(3))
    n_max = 256 * 512
    ramp = (torch.arange(n_max, device=DEV) % 2048).to(torch.float16)
    out = torch.full((n_max,), -1, dtype=torch.float16, device=DEV)
    assert lib.tcx_chunked_roundtrip(case, swizzled, _p(ramp), _p(out), ctypes.byref(rows), ctypes.byref(cols), ctypes.byref(cm)) == 0
    torch.cuda.synchronize()
    n = rows.value * cols.value
    assert torch.equal(out[:n], ramp[:n])
    assert (out[n:] == -1).all()


@pytest.mark.parametrize("case", range(43))
def test_tile_gemm_matches_oracle(lib, case):
    a_buf = torch.zeros(128 * 512, dtype=torch.float16, device=DEV)
    b_buf = torch.zeros(256 * 512, dtype=torch.float16, device=DEV)
    c_buf = torch.full((128 * 256,), float("nan"), device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    m, n, k = (ctypes.c_int() for _ in range(3))
    # learn the shape from a dry call on zeros
    assert lib.tcx_tile_gemm(case, _p(a_buf), _p(b_buf), _p(c_buf), _p(status), ctypes.byref(m), ctypes.byref(n), ctypes.byref(k)) == 0
    torch.cuda.synchronize()
    M, N, K = m.value, n.value, k.value
    a, b = oracle.gemm_inputs(M, N, K, seed=100 + case)
    c = torch.full((M, N), float("nan"), device=DEV)
    a_dev, b_dev = a.to(DEV), b.to(DEV)   # named, so that they outlive the launch
    assert lib.tcx_tile_gemm(case, _p(a_dev), _p(b_dev), _p(c), _p(status), ctypes.byref(m), ctypes.byref(n), ctypes.byref(k)) == 0
    torch.cuda.synchronize()
    assert status.item() == 0
    ref = oracle.gemm(a, b)
    assert oracle.max_abs_err(c, ref) <= 1e-3 and oracle.rel_fro_err(c, ref) <= 1e-5, (M, N, K)


@pytest.mark.parametrize("case", range(3))
def test_tile_b2b_matches_oracle(lib, case):
    dims = [(64, 64, 64, 64), (128, 128, 128, 128), (32, 128, 64, 48)][case]
    M, N, K, P = dims
    a, b, d = oracle.b2b_inputs(M, N, K, P, 1, seed=200 + case)
    e = torch.full((M, P), float("nan"), device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    m, n, k, p = (ctypes.c_int() for _ in range(4))
    a_dev, b_dev, d_dev = a[0].to(DEV), b[0].to(DEV), d[0].to(DEV)   # named, so that they outlive the launch
    rc = lib.tcx_tile_b2b(case, _p(a_dev), _p(b_dev), _p(d_dev), _p(e), _p(status), ctypes.byref(m),
                          ctypes.byref(n), ctypes.byref(k), ctypes.byref(p))
    torch.cuda.synchronize()
    assert rc == 0 and status.item() == 0 and (m.value, n.value, k.value, p.value) == dims
    assert oracle.within_tolerance(e, oracle.back2back_gemm(a[0], b[0], d[0]))


@pytest.mark.parametrize("case", range(6))
def test_tile_flash_attention_matches_oracle(lib, case, golden_dir):
    """Flash attention written with the tile vocabulary (GTileIterator over KV blocks, compute::gemm into TMEM,
    MaxReduce / SumReduce / Broadcast* / RegTileExp for the reference's recurrence). Cases 0-2 are the reference's
    three shapes on its own test inputs, checked against the output of its Python oracle as well."""
    assert lib.tcx_tile_flash_attn_case_count() == 6
    dims = [(64, 64, 128, 128), (64, 128, 128, 128), (64, 256, 128, 128), (128, 512, 128, 128), (128, 256, 64, 64),
            (32, 128, 32, 48)][case]
    M, N, K, P = dims
    golden = None
    if case < 3:
        g = np.load(golden_dir / f"flash_attn_ref_n{N}.npz")
        q, k, v = torch.from_numpy(g["q"]), torch.from_numpy(g["k_t"]).t().contiguous(), torch.from_numpy(g["v"])
        golden = torch.from_numpy(g["o"])
    else:
        q4, k4, v4 = oracle.attention_inputs(1, 1, M, N, K, P, seed=300 + case)
        q, k, v = q4[0, 0], (k4[0, 0].float() * 0.3).half(), v4[0, 0]
    qd, kd, vtd = q.to(DEV).contiguous(), k.to(DEV).contiguous(), v.to(DEV).t().contiguous()
    o = torch.full((M, P), float("nan"), device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    m, n, kk, p = (ctypes.c_int() for _ in range(4))
    rc = lib.tcx_tile_flash_attn(case, _p(qd), _p(kd), _p(vtd), _p(o), _p(status), ctypes.byref(m), ctypes.byref(n),
                                 ctypes.byref(kk), ctypes.byref(p))
    torch.cuda.synchronize()
    assert rc == 0 and status.item() == 0 and (m.value, n.value, kk.value, p.value) == dims
    ref, _ = oracle.flash_attention(q, k, v, scale=1.0)
    assert oracle.within_tolerance(o, ref)
    if golden is not None:
        assert oracle.max_abs_err(o, golden) <= 2e-2


@pytest.mark.parametrize("cols", [16, 64, 128])
def test_row_operations(lib, cols):
    g = torch.Generator().manual_seed(42)                       # test_softmax.cu:86-91: uniform[-5, 5), seed 42
    x = (torch.rand(128, cols, generator=g) * 10 - 5)
    xd = x.to(DEV)
    soft = torch.empty(128, cols, device=DEV)
    centered = torch.empty(128, cols, device=DEV)
    rmax = torch.empty(128, device=DEV)
    rsum = torch.empty(128, device=DEV)
    csum = torch.empty(4, cols, device=DEV)
    assert lib.tcx_row_ops(cols, _p(xd), _p(soft), _p(rmax), _p(rsum), _p(centered), _p(csum)) == 0
    torch.cuda.synchronize()
    assert torch.allclose(soft.cpu(), torch.softmax(x, dim=1), atol=1e-3)   # the reference's bound (test_softmax.cu:113)
    assert torch.equal(rmax.cpu(), x.max(dim=1).values)
    assert torch.allclose(rsum.cpu(), x.sum(dim=1), atol=1e-4)
    assert torch.allclose(centered.cpu(), x - x.max(dim=1, keepdim=True).values, atol=1e-6)
    assert torch.allclose(csum.cpu(), x.view(4, 32, cols).sum(dim=1), atol=1e-4)


@pytest.mark.parametrize("case", range(6))
def test_tile_gemm_over_shared_tile_iterators(lib, case):
    """compute::gemm on the chunks an STileIterator hands out: the shared K slab of each global chunk is multiplied
    in narrower steps, the inner loop of the reference's GEMM example
    (examples/cpp/01_gemm/02_gemm_all_mem/gemm.hpp:145-150)."""
    assert lib.tcx_siter_gemm_case_count() == 6
    dims = [(64, 256, 256), (128, 128, 256), (128, 64, 128), (64, 64, 128), (128, 128, 128), (32, 48, 256)][case]
    M, N, K = dims
    a, b = oracle.gemm_inputs(M, N, K, seed=400 + case)
    c = torch.full((M, N), float("nan"), device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    m, n, k = (ctypes.c_int() for _ in range(3))
    a_dev, b_dev = a.to(DEV), b.to(DEV)
    assert lib.tcx_tile_gemm_siter(case, _p(a_dev), _p(b_dev), _p(c), _p(status), ctypes.byref(m), ctypes.byref(n), ctypes.byref(k)) == 0
    torch.cuda.synchronize()
    assert status.item() == 0 and (m.value, n.value, k.value) == dims
    ref = oracle.gemm(a, b)
    assert oracle.max_abs_err(c, ref) <= 1e-3 and oracle.rel_fro_err(c, ref) <= 1e-5, dims


@pytest.mark.parametrize("case", range(6))
def test_shared_to_reg_loader_round_trip(lib, case):
    """global -> shared operand tile (swizzled or interleaved) -> SharedToRegLoader (one row per thread, fp16 kept or
    widened to fp32) -> global reproduces the `i % 2048` ramp exactly."""
    assert lib.tcx_shared_to_reg_case_count() == 6
    rows, cols, elem = (ctypes.c_int() for _ in range(3))
    ramp = (torch.arange(128 * 128, device=DEV) % 2048).to(torch.float16)
    out = torch.full((128 * 128,), -1.0, dtype=torch.float32, device=DEV)
    assert lib.tcx_shared_to_reg(case, _p(ramp), _p(out), ctypes.byref(rows), ctypes.byref(cols), ctypes.byref(elem)) == 0
    torch.cuda.synchronize()
    n = rows.value * cols.value
    got = out.view(torch.float16)[:n] if elem.value == 2 else out[:n]
    assert torch.equal(got.float(), ramp[:n].float())


@pytest.mark.parametrize("cols", [16, 64, 128])
def test_reg_to_tmem_storer_round_trip(lib, cols):
    """row fragments -> RegToTmemStorer -> tensor memory -> TmemToRegLoader -> global is exact."""
    x = torch.randn(128, cols, generator=torch.Generator().manual_seed(7)).to(DEV)
    y = torch.full_like(x, float("nan"))
    assert lib.tcx_tmem_roundtrip(cols, _p(x), _p(y)) == 0
    torch.cuda.synchronize()
    assert torch.equal(x, y)


@pytest.mark.parametrize("case,row0,col0", [(0, 0, 0), (0, 64, 128), (1, 128, 64), (2, 32, 0), (1, 200, 192)])
def test_tma_tile_loader_matches_the_matrix(lib, case, row0, col0):
    """TmaTileLoader: a tensor map built on the host, one thread issuing the loads into a swizzled operand tile; the
    tile read back through SharedToGlobalStorer equals the same window of the matrix (what the cp.async loader
    delivers), with zero fill where the window leaves the matrix."""
    rows, cols = 256, 320
    src = (torch.arange(rows * cols, device=DEV) % 2048).to(torch.float16).view(rows, cols)
    tr, tc = [(64, 64), (128, 128), (32, 256)][case]
    out = torch.full((tr, tc), -1.0, dtype=torch.float16, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    r, c = ctypes.c_int(), ctypes.c_int()
    assert lib.tcx_tma_load(case, _p(src), rows, cols, row0, col0, _p(out), _p(status), ctypes.byref(r), ctypes.byref(c)) == 0
    torch.cuda.synchronize()
    assert status.item() == 0 and (r.value, c.value) == (tr, tc)
    want = torch.zeros(tr, tc, dtype=torch.float16, device=DEV)
    rr, cc = min(tr, rows - row0), min(tc, cols - col0)
    want[:rr, :cc] = src[row0:row0 + rr, col0:col0 + cc]
    assert torch.equal(out, want)


def test_a_wait_that_runs_out_returns_a_status_and_leaves_the_device_usable(lib):
    """A bounded wait gives up: a CTA waits 2 ms on an MMA barrier that nothing commits, reports status 1, frees its
    tensor memory and returns (no trap, no endless loop). The next kernel on the same context runs normally."""
    status = torch.full((1,), -1, dtype=torch.int32, device=DEV)
    waited = torch.zeros(1, dtype=torch.int64, device=DEV)
    lib.tcx_wait_runs_out.argtypes = [ctypes.c_ulonglong, ctypes.c_void_p, ctypes.c_void_p]
    assert lib.tcx_wait_runs_out(2_000_000, _p(status), _p(waited)) == 0
    torch.cuda.synchronize()
    assert status.item() == 1
    assert 2_000_000 <= waited.item() < 200_000_000   # gave up after the limit, and soon after it
    # the context is intact: a tile GEMM (which allocates the tensor memory the waiting CTA freed) still matches
    a, b = oracle.gemm_inputs(128, 128, 64, seed=9)
    c = torch.full((128, 128), float("nan"), device=DEV)
    st = torch.zeros(1, dtype=torch.int32, device=DEV)
    m, n, k = (ctypes.c_int() for _ in range(3))
    a_dev, b_dev = a.to(DEV), b.to(DEV)
    assert lib.tcx_tile_gemm(12, _p(a_dev), _p(b_dev), _p(c), _p(st), ctypes.byref(m), ctypes.byref(n), ctypes.byref(k)) == 0
    torch.cuda.synchronize()
    assert st.item() == 0 and oracle.max_abs_err(c, oracle.gemm(a, b)) <= 1e-3
