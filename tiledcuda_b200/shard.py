"""Data-parallel sharding of the tile-kernel ops across the GPUs of one box, one process per GPU.

The reference is single-GPU. Every op on this path consists of independent units (GEMM row slabs,
(batch, head) pairs of attention, batch rows of the LSTM, owned row ranges of the scatter table),
so a rank computes a contiguous range of units with no communication on the data path. The only
collective is an optional all-gather (NCCL over NVLink on GPUs, gloo in CPU tests) that assembles
the full output on every rank.
"""
from __future__ import annotations

from typing import Callable, Tuple

import torch
import torch.distributed as dist


def shard_range(total: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous, balanced [start, stop) of `total` units for `rank` of `world` (first ranks get the remainder)."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError(f"bad rank {rank} of world {world}")
    if total < 0:
        raise ValueError("total must be non-negative")
    base, rem = divmod(total, world)
    start = rank * base + min(rank, rem)
    return start, start + base + (1 if rank < rem else 0)


def aligned_shard_range(total: int, world: int, rank: int, align: int) -> Tuple[int, int]:
    """As shard_range, but every boundary except the last is a multiple of `align` (e.g. the 128-row tile)."""
    blocks = (total + align - 1) // align
    b0, b1 = shard_range(blocks, world, rank)
    return min(b0 * align, total), min(b1 * align, total)


def all_gather_slabs(full: torch.Tensor, world: int, rank: int, ranges=None, group=None) -> None:
    """Completes `full` (first dimension = units) on every rank; each rank has already written its own slab.

    Equal slabs use one in-place all_gather_into_tensor; ragged ones fall back to a broadcast per rank.
    """
    total = full.shape[0]
    if ranges is None:
        ranges = [shard_range(total, world, r) for r in range(world)]
    if world == 1:
        return
    sizes = {b - a for a, b in ranges}
    start, stop = ranges[rank]
    if len(sizes) == 1 and full.is_contiguous():
        dist.all_gather_into_tensor(full, full[start:stop], group=group)
        return
    for r, (a, b) in enumerate(ranges):
        if b > a:
            dist.broadcast(full[a:b], src=r, group=group)


def run_sharded(
    total_units: int,
    compute: Callable[[int, int], None],
    full_output: torch.Tensor | None = None,
    gather: bool = False,
    align: int = 1,
    group=None,
) -> Tuple[int, int]:
    """Runs `compute(start, stop)` on this rank's unit range, then optionally all-gathers `full_output`.

    `compute` writes units [start, stop) of the output (normally straight into a view of
    `full_output`). Without an initialised process group this is the whole range on one rank.
    """
    if dist.is_available() and dist.is_initialized():
        world, rank = dist.get_world_size(group), dist.get_rank(group)
    else:
        world, rank = 1, 0
    ranges = [aligned_shard_range(total_units, world, r, align) for r in range(world)]
    start, stop = ranges[rank]
    if stop > start:
        compute(start, stop)
    if gather and full_output is not None:
        all_gather_slabs(full_output, world, rank, ranges, group)
    return start, stop


def sharded_gemm(a: torch.Tensor, b: torch.Tensor, c: torch.Tensor, gather: bool = True, group=None) -> Tuple[int, int]:
    """c = a @ b.T with the rows of a (and c) split across ranks; b is replicated."""
    from . import ops

    def compute(start: int, stop: int) -> None:
        ops.gemm(a[start:stop], b, c[start:stop])

    return run_sharded(a.shape[0], compute, c, gather, align=128, group=group)


def sharded_flash_attn(q, k, v, o, scale=None, gather: bool = True, group=None) -> Tuple[int, int]:
    """Attention with the (batch x heads) pairs split across ranks; tensors are [B, H, S, D]."""
    from . import ops

    b, h = q.shape[:2]
    qf, kf, vf, of = (t.view(1, b * h, *t.shape[2:]) for t in (q, k, v, o))

    def compute(start: int, stop: int) -> None:
        ops.flash_attn(qf[:, start:stop], kf[:, start:stop], vf[:, start:stop], of[:, start:stop], scale=scale)

    return run_sharded(b * h, compute, of[0], gather, group=group)


def sharded_lstm_chain(w, u, bias, x, h0, c0, h_all, c_out, gather: bool = True, group=None) -> Tuple[int, int]:
    """LSTM chain with the batch rows split across ranks (weights replicated); x is [T, B, I]."""
    from . import ops

    def compute(start: int, stop: int) -> None:
        xs = x[:, start:stop].contiguous()
        hs = torch.empty(x.shape[0], stop - start, h_all.shape[2], dtype=h_all.dtype, device=h_all.device)
        ops.lstm_chain(w, u, bias, xs, h0[start:stop], c0[start:stop], hs, c_out[start:stop])
        h_all[:, start:stop].copy_(hs)

    rng = run_sharded(x.shape[1], compute, None, False, group=group)
    if gather:
        world = dist.get_world_size(group) if dist.is_initialized() else 1
        rank = dist.get_rank(group) if dist.is_initialized() else 0
        ranges = [shard_range(x.shape[1], world, r) for r in range(world)]
        all_gather_slabs(c_out, world, rank, ranges, group)
        hb = h_all.transpose(0, 1).contiguous()
        all_gather_slabs(hb, world, rank, ranges, group)
        h_all.copy_(hb.transpose(0, 1))
    return rng


def sharded_scatter_nd(table_slab: torch.Tensor, row_start: int, indices: torch.Tensor, updates: torch.Tensor) -> int:
    """Owner-computes scatter: this rank holds table rows [row_start, row_start + len(slab)) and applies
    only the updates that fall into them. indices is [n, 1]. Returns the number of rows applied here."""
    from . import ops

    rows = indices.view(-1)
    mine = (rows >= row_start) & (rows < row_start + table_slab.shape[0])
    local_idx = (rows[mine] - row_start).to(indices.dtype).view(-1, 1).contiguous()
    local_upd = updates[mine].contiguous()
    if local_idx.numel():
        ops.scatter_nd(table_slab, local_idx, local_upd)
    return int(local_idx.shape[0])
