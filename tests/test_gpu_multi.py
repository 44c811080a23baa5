"""Two NCCL ranks on two GPUs: every partition of tiledcuda_b200/shard.py (GEMM rows, attention (batch, head)
pairs, LSTM batch rows, owner-computes scatter_nd), the overlapped assembly of C and the host-operand pipeline,
each compared with the CPU oracle after the gather. Skipped on a box with fewer than two GPUs; the same
partitioning logic runs on two gloo ranks on the CPU in tests/test_host_logic.py."""
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    import torch.distributed as dist

    from oracle import oracle
    from tiledcuda_b200 import _lib, ops, shard

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    ok = {}
    try:
        # GEMM: rows split, C gathered; then the overlapped form (row blocks exchanged while later ones compute)
        a, b = oracle.gemm_inputs(2048, 640, 512)
        want = oracle.gemm(a, b)
        a_d, b_d = a.to(dev), b.to(dev)
        c = torch.full((2048, 640), float("nan"), device=dev)
        shard.sharded_gemm(a_d, b_d, c, gather=True)
        torch.cuda.synchronize()
        ok["gemm"] = oracle.within_tolerance(c, want, 2e-3, 1e-5)
        c2 = torch.full((2048, 640), float("nan"), device=dev)
        shard.OverlappedGemm(blocks=4, max_sms=132)(a_d, b_d, c2)
        torch.cuda.synchronize()
        ok["gemm_overlapped"] = bool(torch.equal(c2, c))
        c3 = torch.full((2048, 640), float("nan"), device=dev)
        push = shard.OverlappedGemm(blocks=4, transport="copy_engine")
        push(a_d, b_d, c3)
        torch.cuda.synchronize()
        ok["gemm_overlapped_copy_engine"] = bool(torch.equal(c3, c))
        c3.fill_(float("nan"))
        dist.barrier()                       # nobody pushes into a C that is still being poisoned
        push(a_d, b_d, c3)                   # second call: the windows are reused
        torch.cuda.synchronize()
        ok["gemm_overlapped_copy_engine_again"] = bool(torch.equal(c3, c))
        push.assembly.windows.close()        # windows are closed before their tensors are freed
        dist.barrier()

        # the host-operand pipeline: own A slab and half of B from the host, B gathered over NVLink
        pipe = shard.HostGemmPipeline(1024, 640, 512, dev, blocks=4)
        lo, hi = pipe.b_slice()
        h_c = torch.empty(1024, 640).pin_memory()
        pipe(a[rank * 1024:(rank + 1) * 1024].pin_memory(), b[lo:hi].pin_memory(), h_c)
        torch.cuda.synchronize()
        ok["gemm_host"] = bool(torch.equal(h_c, c[rank * 1024:(rank + 1) * 1024].cpu()))

        # attention over (batch, head) pairs
        q_, k_, v_ = oracle.attention_inputs(2, 3, 256, 320, 64)
        o = torch.full((2, 3, 256, 64), float("nan"), dtype=torch.float16, device=dev)
        shard.sharded_flash_attn(q_.to(dev), k_.to(dev), v_.to(dev), o, gather=True)
        torch.cuda.synchronize()
        ok["fa"] = oracle.within_tolerance(o, oracle.flash_attention(q_, k_, v_)[0])
        o2 = torch.full((2, 3, 256, 64), float("nan"), dtype=torch.float16, device=dev)
        assembly = shard.OverlappedAssembly(blocks=2)
        shard.overlapped_flash_attn(assembly, q_.to(dev), k_.to(dev), v_.to(dev), o2)
        torch.cuda.synchronize()
        ok["fa_overlapped"] = bool(torch.equal(o2, o))
        assembly.windows.close()
        dist.barrier()

        # LSTM chain over batch rows
        w, u, bias, x, h0, c0 = oracle.lstm_inputs(5, 192, 128, 64, with_bias=True)
        h_all = torch.full((5, 192, 64), float("nan"), dtype=torch.float16, device=dev)
        c_t = torch.full((192, 64), float("nan"), device=dev)
        shard.sharded_lstm_chain(w.to(dev), u.to(dev), bias.to(dev), x.to(dev), h0.to(dev), c0.to(dev), h_all, c_t, gather=True)
        torch.cuda.synchronize()
        rh, rc = oracle.lstm_chain(w, u, bias, x, h0, c0)
        ok["lstm"] = oracle.within_tolerance(h_all, rh) and oracle.within_tolerance(c_t, rc)

        # scatter_nd: each rank owns half of the table rows
        table, idx, upd = oracle.scatter_inputs(4096, 8, 1500)
        r0, r1 = shard.shard_range(4096, world, rank)
        full = torch.zeros(4096, 8, dtype=table.dtype, device=dev)
        full[r0:r1] = table[r0:r1].to(dev)
        applied = shard.sharded_scatter_nd(full[r0:r1], r0, idx.to(dev), upd.to(dev))
        shard.all_gather_slabs(full, world, rank)
        torch.cuda.synchronize()
        want_t = oracle.scatter_nd(table.numpy(), idx.numpy(), upd.numpy())
        ok["scatter"] = full.cpu().numpy().tobytes() == want_t.tobytes() and 0 < applied < 1500
        ok["status"] = _lib.device_status() == 0
        q.put((rank, ok))
    finally:
        dist.destroy_process_group()


def test_two_nccl_ranks_shard_gather_and_match_the_oracle():
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = sorted(q.get(timeout=300) for _ in procs)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    for rank, ok in results:
        assert all(ok.values()), (rank, ok)
