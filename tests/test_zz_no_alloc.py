"""GPU test of the entry point that allocates nothing, tc_lstm_chain_static_f16.

Who needs it: callers that cannot call cudaMalloc where they run the chain (inside a stream capture,
in a loop whose device memory was fixed at start-up, or a plug-in that only gets input and output
buffers) and so cannot give tc_lstm_chain_ws_f16 the workspace it asks for. The entry point keeps that
workspace in a 64 MiB array inside the library image instead.

The test goes through the C ABI with ctypes, runs the entry point twice in a row on different inputs
(the array keeps the first call's contents, which the second call must fully overwrite) and compares each
result with tc_lstm_chain_ws_f16 on the same inputs: same kernels, same order of operations, so the
outputs must agree to the bit; the assertion allows the tolerance the other LSTM tests use. Around the
second problem's calls it reads the free device memory (cudaMemGetInfo) and requires it unchanged: the call
allocated nothing. It also checks the size limit and the steps == 0 status query. The file name sorts after every other test file
so that a run that stops at the first failure has already run the rest.
"""
import ctypes

import pytest
import torch

from oracle import oracle

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
STATIC_SCRATCH_BYTES = 64 * 1024 * 1024


def _ptr(t):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _free_device_bytes():
    """Free device memory as the driver reports it (cudaMemGetInfo), past torch's caching allocator."""
    free, _total = torch.cuda.mem_get_info(0)
    return free


def _run_static(lib, w, u, bias, x, h0, c0, h_all, c_out):
    steps, batch, inp = x.shape
    hidden = u.shape[1]
    return lib.tc_lstm_chain_static_f16(_ptr(w), _ptr(u), _ptr(bias), _ptr(x), _ptr(h0), _ptr(c0), _ptr(h_all), _ptr(c_out),
                                        steps, batch, inp, hidden, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))


def _run_workspace(lib, w, u, bias, x, h0, c0, h_all, c_out):
    steps, batch, inp = x.shape
    hidden = u.shape[1]
    ws = torch.empty(lib.tc_lstm_chain_workspace_bytes(steps, batch, hidden) // 4, device=DEV)
    rc = lib.tc_lstm_chain_ws_f16(_ptr(w), _ptr(u), _ptr(bias), _ptr(x), _ptr(h0), _ptr(c0), _ptr(h_all), _ptr(c_out),
                                  steps, batch, inp, hidden, _ptr(ws), ws.numel() * 4,
                                  ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    return rc


def test_static_scratch_chain_matches_the_workspace_chain_twice_in_a_row():
    assert torch.cuda.is_available()
    from tiledcuda_b200 import _lib

    lib = _lib.load()
    torch.cuda.set_device(0)
    # two different problems, the second smaller than the first, so stale scratch from call one lies
    # beyond (and, if the GEMM did not overwrite it, inside) what call two reads
    for steps, batch, inp, hidden, seed in ((12, 256, 512, 512, 11), (7, 200, 264, 496, 12)):
        w, u, bias, x, h0, c0 = oracle.lstm_inputs(steps, batch, inp, hidden, seed=seed, with_bias=True)
        g = torch.Generator().manual_seed(seed)
        h0 = (torch.randn(batch, hidden, generator=g) * 0.5).half()
        c0 = torch.randn(batch, hidden, generator=g)
        dev = [t.to(DEV) for t in (w, u, bias, x, h0, c0)]
        h_static = torch.full((steps, batch, hidden), float("nan"), dtype=torch.float16, device=DEV)
        c_static = torch.full((batch, hidden), float("nan"), device=DEV)
        rc = _run_static(lib, *dev, h_static, c_static)
        assert rc == 0, lib.tc_last_error().decode()
        torch.cuda.synchronize()
        # The claim in the entry point's name: a call takes no device memory. Free memory as the driver reports it
        # (cudaMemGetInfo) is read on both sides of a second call with the same shapes; the first call with a shape
        # class may make the driver load kernels, which is not an allocation of the entry point's.
        h_first, c_first = h_static.clone(), c_static.clone()   # computed over whatever the previous problem left in the scratch
        free_before = _free_device_bytes()
        h_static.fill_(float("nan"))
        c_static.fill_(float("nan"))
        rc = _run_static(lib, *dev, h_static, c_static)
        assert rc == 0, lib.tc_last_error().decode()
        torch.cuda.synchronize()
        assert _free_device_bytes() == free_before
        assert torch.equal(h_first, h_static) and torch.equal(c_first, c_static)
        h_ws = torch.empty_like(h_static)
        c_ws = torch.empty_like(c_static)
        assert _run_workspace(lib, *dev, h_ws, c_ws) == 0, lib.tc_last_error().decode()
        assert oracle.max_abs_err(h_static, h_ws) <= oracle.MAX_ABS_TOL and oracle.rel_fro_err(h_static, h_ws) <= oracle.REL_FRO_TOL
        assert oracle.max_abs_err(c_static, c_ws) <= oracle.MAX_ABS_TOL and oracle.rel_fro_err(c_static, c_ws) <= oracle.REL_FRO_TOL
        rh, rc_ref = oracle.lstm_chain(w, u, bias, x, h0, c0)
        assert oracle.within_tolerance(h_static, rh) and oracle.within_tolerance(c_static, rc_ref)
    # steps == 0: status query of this path, nothing recorded
    none = ctypes.c_void_p(0)
    assert lib.tc_lstm_chain_static_f16(none, none, none, none, none, none, none, none, 0, 1, 8, 16, none) == 0


def test_static_scratch_chain_rejects_sizes_beyond_its_array():
    from tiledcuda_b200 import _lib

    lib = _lib.load()
    torch.cuda.set_device(0)
    steps, batch, inp, hidden = 64, 256, 64, 1024  # 64 * 256 * 4096 * 4 bytes = 256 MiB of scratch
    assert steps * batch * 4 * hidden * 4 > STATIC_SCRATCH_BYTES
    w = torch.zeros(4 * hidden, inp, dtype=torch.float16, device=DEV)
    u = torch.zeros(4 * hidden, hidden, dtype=torch.float16, device=DEV)
    x = torch.zeros(steps, batch, inp, dtype=torch.float16, device=DEV)
    h0 = torch.zeros(batch, hidden, dtype=torch.float16, device=DEV)
    c0 = torch.zeros(batch, hidden, device=DEV)
    h_all = torch.zeros(steps, batch, hidden, dtype=torch.float16, device=DEV)
    c_out = torch.zeros(batch, hidden, device=DEV)
    rc = _run_static(lib, w, u, None, x, h0, c0, h_all, c_out)
    assert rc == -2  # TC_ERR_UNSUPPORTED
    msg = lib.tc_last_error().decode()
    assert "exceed" in msg and "67108864" in msg
