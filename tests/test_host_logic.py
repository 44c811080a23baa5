"""CPU tests of the host side: the op wrappers refuse anything that is not a CUDA tensor of the
right dtype and shape (there is no CPU fallback), and the sharding logic partitions and reassembles
correctly, including on two gloo ranks."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import oracle
from tiledcuda_b200 import ops, shard


def test_ops_refuse_cpu_tensors():
    a = torch.zeros(128, 64, dtype=torch.float16)
    c = torch.zeros(128, 128)
    with pytest.raises(ValueError, match="CUDA"):
        ops.gemm(a, a, c)
    with pytest.raises(ValueError, match="CUDA"):
        ops.scatter_nd(torch.zeros(4, 4), torch.zeros(1, 1, dtype=torch.int64), torch.zeros(1, 4))
    q = torch.zeros(1, 1, 128, 64, dtype=torch.float16)
    with pytest.raises(ValueError, match="CUDA"):
        ops.flash_attn(q, q, q, q)
    with pytest.raises(ValueError, match="CUDA"):
        ops.lstm_cell(a, a, None, a, a, c, a, c)


def test_product_package_does_not_import_the_oracle():
    import pathlib
    import re

    pkg = pathlib.Path(ops.__file__).parent
    for f in list(pkg.glob("*.py")) + list(pkg.glob("csrc/*")):
        text = f.read_text(errors="ignore")
        assert not re.search(r"^\s*(from|import)\s+oracle\b", text, flags=re.M), f


@pytest.mark.parametrize("total,world", [(0, 1), (1, 4), (7, 3), (512, 8), (64, 8), (10, 4)])
def test_shard_range_partitions_exactly(total, world):
    ranges = [shard.shard_range(total, world, r) for r in range(world)]
    assert ranges[0][0] == 0 and ranges[-1][1] == total
    for (a0, a1), (b0, b1) in zip(ranges, ranges[1:]):
        assert a1 == b0 and a0 <= a1
    sizes = [b - a for a, b in ranges]
    assert max(sizes) - min(sizes) <= 1


def test_aligned_shard_range_keeps_tile_boundaries():
    ranges = [shard.aligned_shard_range(1000, 3, r, 128) for r in range(3)]
    assert ranges[0][0] == 0 and ranges[-1][1] == 1000
    for a, b in ranges[:-1]:
        assert a % 128 == 0 and b % 128 == 0
    with pytest.raises(ValueError):
        shard.shard_range(4, 2, 2)


def test_run_sharded_single_rank_covers_everything():
    seen = []
    shard.run_sharded(10, lambda a, b: seen.append((a, b)))
    assert seen == [(0, 10)]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _gloo_worker(rank, world, port, ragged, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        m = 300 if ragged else 256
        a, b = oracle.gemm_inputs(m, 48, 64)
        c = torch.zeros(m, 48)

        # the oracle stands in for the kernel here: this test is about partitioning and gathering
        def compute(start, stop):
            c[start:stop] = oracle.gemm(a[start:stop], b)

        start, stop = shard.run_sharded(m, compute, c, gather=True, align=128)
        ok_gather = torch.equal(c, oracle.gemm(a, b))

        # scatter ownership: each rank applies only its rows; together they equal the oracle
        table, idx, upd = oracle.scatter_inputs(64, 8, 40)
        r0, r1 = shard.shard_range(64, world, rank)
        rows = idx.view(-1)
        mine = (rows >= r0) & (rows < r1)
        slab = table[r0:r1].clone()
        slab[(rows[mine] - r0).long()] = upd[mine]
        full = torch.zeros_like(table)
        full[r0:r1] = slab
        shard.all_gather_slabs(full, world, rank)
        want = torch.from_numpy(oracle.scatter_nd(table.numpy(), idx.numpy(), upd.numpy()))

        # block-wise assembly (what the overlapped GEMM does per finished row block): each rank fills its own
        # slab, then the slabs are exchanged two row blocks at a time with grouped send / receive
        if not ragged:
            ranges = [shard.aligned_shard_range(m, world, r, 128) for r in range(world)]
            c2 = torch.zeros(m, 48)
            s2, e2 = ranges[rank]
            c2[s2:e2] = oracle.gemm(a[s2:e2], b)
            half = (e2 - s2) // 2
            for lo, hi in ((0, half), (half, e2 - s2)):
                for w in shard.exchange_row_block(c2, ranges, lo, hi):
                    w.wait()
            ok_gather = ok_gather and torch.equal(c2, oracle.gemm(a, b))
        q.put((rank, start, stop, bool(ok_gather), bool(torch.equal(full, want))))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("ragged", [False, True])
def test_two_gloo_ranks_shard_and_gather(ragged):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_gloo_worker, args=(r, 2, port, ragged, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert results[0][1] == 0 and results[0][2] == results[1][1]
    assert results[1][2] == (300 if ragged else 256)
    assert all(r[3] and r[4] for r in results)


def test_torch_op_library_registers_the_reference_ops_and_has_no_cpu_kernel():
    from tiledcuda_b200 import pytiledcuda

    for name in ("scatter_nd", "flash_attention_fwd", "gemm", "back2back_gemm", "lstm_cell", "flash_attn"):
        assert hasattr(torch.ops.tiledcuda, name)
    a = torch.zeros(8, 8, dtype=torch.float16)
    with pytest.raises((NotImplementedError, RuntimeError)):
        pytiledcuda.gemm(a, a, torch.zeros(8, 8))
    for name in ("scatter_nd", "flash_attention_fwd", "TiledFlashAttention"):
        assert hasattr(pytiledcuda, name)
    # and under the reference's own package name
    import pytiledcuda as by_reference_name

    assert by_reference_name.TiledFlashAttention is pytiledcuda.TiledFlashAttention
    assert by_reference_name.scatter_nd is pytiledcuda.scatter_nd
