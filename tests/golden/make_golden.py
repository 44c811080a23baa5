"""Generates the golden fixtures in this directory. Run once, in a container where the reference
checkout is mounted:

    python tests/golden/make_golden.py [/path/to/reference]

Sources of the vectors:
  flash_attn_ref_n{64,128,256}.npz   the reference's own Python oracle class `FlashAttention`
      (tests/python/test_flash_attn.py:9-75), imported from the reference tree and run on the inputs its
      test draws (seed 1234, shapes :124-161). Its output buffer is zero-filled before forward(),
      because the class starts from torch.empty and multiplies that by zero (:25, :67).
  scatter_nd_ref.npz                 the reference test's setup (tests/python/test_scatter_nd.py:22-41: data
      [7,8,9,10] filled 5.0, five (i, j) pairs, updates filled 10.0) and its oracle statement
      `data[indices[:, 0], indices[:, 1]] = updates` (:46), executed here with torch; the reference
      draws the pairs from unseeded `random`, here seeded with 1234. A second case uses random values
      and unique rows.
  gemm_ramp.npz                      inputs `i % 2048 / 1000` and the naive fp32 triple loop of
      tests/cpp/cell/test_single_wmma.cu:16-29, 58-62, written out as Python loops over float32.
  lstm_cell_torch.npz                torch.nn.LSTMCell (fp32, CPU) on fp16-representable values; the reference
      snapshot has no LSTM code to take vectors from.
The fixtures are read by tests/ only.
"""
from __future__ import annotations

import importlib.util
import random
import sys
import types
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def load_reference_flash_attention(ref_root: Path):
    """Imports tests/python/test_flash_attn.py from the reference with its GPU-only imports stubbed."""
    sys.modules.setdefault("context", types.ModuleType("context"))
    stub = types.ModuleType("pytiledcuda")
    stub.TiledFlashAttention = None
    sys.modules["pytiledcuda"] = stub
    spec = importlib.util.spec_from_file_location("ref_test_flash_attn", ref_root / "tests/python/test_flash_attn.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.FlashAttention


def make_flash_attn(ref_root: Path) -> None:
    FlashAttention = load_reference_flash_attention(ref_root)
    m, k, p = 64, 128, 128
    for n in (64, 128, 256):
        torch.manual_seed(1234)
        q = torch.randn(m, k)
        kt = torch.randn(k, n)
        v = torch.randn(n, p)
        fa = FlashAttention(q.half().flatten(), kt.half().flatten(), v.half().flatten(), m, n, k, p, 64, 64, 128, 128)
        fa.output = torch.zeros(m, p)
        ref_o = fa.forward().half()
        assert torch.isfinite(ref_o.float()).all()
        np.savez(
            HERE / f"flash_attn_ref_n{n}.npz",
            q=q.half().numpy(), k_t=kt.half().numpy(), v=v.half().numpy(), o=ref_o.numpy(),
            shape=np.array([m, n, k, p, 64, 64, 128, 128]),
        )


def make_scatter() -> None:
    random.seed(1234)
    data_shape = [7, 8, 9, 10]
    data = torch.empty(data_shape, dtype=torch.float32).fill_(5.0)
    indices = torch.empty([5, 2], dtype=torch.int64)
    for i in range(5):
        indices[i][0] = random.randint(0, data_shape[0] - 1)
        indices[i][1] = random.randint(0, data_shape[1] - 1)
    updates = torch.empty([5, 9, 10], dtype=torch.float32).fill_(10.0)
    out = data.clone()
    out[indices[:, 0], indices[:, 1]] = updates

    g = torch.Generator().manual_seed(1234)
    data2 = torch.randn(64, 6, 8, generator=g).half()
    idx2 = torch.randperm(64, generator=g)[:20].view(20, 1)
    upd2 = torch.randn(20, 6, 8, generator=g).half()
    out2 = data2.clone()
    out2[idx2[:, 0]] = upd2
    np.savez(
        HERE / "scatter_nd_ref.npz",
        data=data.numpy(), indices=indices.numpy(), updates=updates.numpy(), out=out.numpy(),
        data2=data2.numpy(), indices2=idx2.numpy(), updates2=upd2.numpy(), out2=out2.numpy(),
    )


def make_gemm_ramp() -> None:
    cases = {}
    for tag, (m, n, k) in {"16": (16, 16, 16), "64x128x128": (64, 128, 128)}.items():
        a = np.array([np.float16((i % 2048) / 1000.0) for i in range(m * k)], dtype=np.float16).reshape(m, k)
        b = np.array([np.float16((i % 2048) / 1000.0) for i in range(n * k)], dtype=np.float16).reshape(n, k)
        c = np.zeros((m, n), dtype=np.float32)
        a32 = a.astype(np.float32)
        b32 = b.astype(np.float32)
        for i in range(m):
            for j in range(n):
                s = np.float32(0.0)
                for kk in range(k):
                    s = np.float32(s + a32[i, kk] * b32[j, kk])
                c[i, j] = s
        cases[f"a_{tag}"] = a
        cases[f"b_{tag}"] = b
        cases[f"c_{tag}"] = c
    np.savez(HERE / "gemm_ramp.npz", **cases)


def make_lstm() -> None:
    torch.manual_seed(1234)
    batch, inp, hidden = 24, 40, 32
    cell = torch.nn.LSTMCell(inp, hidden)
    with torch.no_grad():
        for prm in cell.parameters():
            prm.copy_(prm.half().float())
        x = torch.randn(batch, inp).half().float()
        h = (torch.randn(batch, hidden) * 0.5).half().float()
        c = torch.randn(batch, hidden)
        h1, c1 = cell(x, (h, c))
    np.savez(
        HERE / "lstm_cell_torch.npz",
        w=cell.weight_ih.detach().half().numpy(), u=cell.weight_hh.detach().half().numpy(),
        bias=(cell.bias_ih + cell.bias_hh).detach().numpy(),
        x=x.half().numpy(), h=h.half().numpy(), c=c.numpy(), h1=h1.numpy(), c1=c1.numpy(),
    )


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py <path of the reference checkout>")
    ref = Path(sys.argv[1])
    make_flash_attn(ref)
    make_scatter()
    make_gemm_ramp()
    make_lstm()
    for f in sorted(HERE.glob("*.npz")):
        print(f.name, f.stat().st_size)
