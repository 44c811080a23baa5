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


# ----------------------------------------------------------------------------------------------------
# Assembling C while it is still being computed
# ----------------------------------------------------------------------------------------------------
def exchange_row_block(full: torch.Tensor, ranges, lo: int, hi: int, group=None):
    """Every rank sends rows [start + lo, start + hi) of its own slab of `full` to every other rank and receives
    theirs into place (start = first row of the owner's slab): one grouped send/receive over NVLink, zero-copy on
    both sides because whole rows of `full` are contiguous. Returns the work handles; wait on them (or on the
    stream they were issued from) before reading the received rows. Slabs must be at least `hi` rows long."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    ops_list = []
    mine = full[ranges[rank][0] + lo: ranges[rank][0] + hi]
    for step in range(1, world):
        # send to rank + step while receiving from rank - step: every link is busy in every slot of the schedule
        to, frm = (rank + step) % world, (rank - step) % world
        ops_list.append(dist.P2POp(dist.isend, mine, to, group=group))
        ops_list.append(dist.P2POp(dist.irecv, full[ranges[frm][0] + lo: ranges[frm][0] + hi], frm, group=group))
    return dist.batch_isend_irecv(ops_list) if ops_list else []


# Device allocations of other ranks that this process has opened: handle bytes -> [base address here, users]. An
# allocation is opened once per process however many windows lie in it (the caching allocator packs several
# tensors into one allocation).
_OPENED_PEER_ALLOCATIONS: dict = {}


class PeerWindows:
    """The same tensor of every rank of the box, writable from this rank (one process per GPU, all GPUs of the box
    visible to every process). Each rank exports the device allocation its tensor lies in (tc_peer_export) and opens
    the others' with its own GPU current (tc_peer_open), which maps them with peer access over NVLink. A push is
    a device-to-device cudaMemcpyAsync from local memory into a peer's window: it runs on the copy engines and
    takes no SM from the kernels that run beside it. The exporting rank must keep its tensor alive while any rank
    still holds a window on it."""

    HANDLE_BYTES = 64

    def __init__(self, tensor: torch.Tensor, group=None):
        import ctypes

        from . import _lib

        if not tensor.is_contiguous():
            raise ValueError("peer windows need a contiguous tensor")
        self.lib = _lib.load()
        self.check = _lib.check
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.group = group
        self.tensor = tensor
        self.key = (tensor.data_ptr(), tuple(tensor.shape))
        # offset of the tensor inside its device allocation (the caching allocator's segment)
        base_addr = None
        for seg in torch.cuda.memory_snapshot():
            if seg["device"] == tensor.device.index and seg["address"] <= tensor.data_ptr() < seg["address"] + seg["total_size"]:
                base_addr = seg["address"]
        if base_addr is None:
            raise RuntimeError("the tensor does not lie in a device allocation of this process's caching allocator")
        offset = tensor.data_ptr() - base_addr
        handle = ctypes.create_string_buffer(self.HANDLE_BYTES)
        with torch.cuda.device(tensor.device):
            self.check("tc_peer_export", self.lib.tc_peer_export(ctypes.c_void_p(base_addr), handle, self.HANDLE_BYTES))
            exported = [None] * self.world
            dist.all_gather_object(exported, (handle.raw, offset), group=group)
            self.bases = [None] * self.world
            self.ptrs = [None] * self.world
            for r, (raw, off) in enumerate(exported):
                if r == self.rank:
                    self.ptrs[r] = tensor.data_ptr()
                    continue
                entry = _OPENED_PEER_ALLOCATIONS.get(raw)
                if entry is None:
                    base = ctypes.c_void_p()
                    self.check("tc_peer_open", self.lib.tc_peer_open(ctypes.create_string_buffer(raw, self.HANDLE_BYTES), self.HANDLE_BYTES,
                                                                     ctypes.byref(base)))
                    entry = _OPENED_PEER_ALLOCATIONS[raw] = [base.value, 0]
                entry[1] += 1
                self.bases[r] = raw
                self.ptrs[r] = entry[0] + off
        self.flag = torch.zeros(1, device=tensor.device)
        self.row_bytes = tensor.stride(0) * tensor.element_size()

    def push_rows(self, lo: int, hi: int, streams=None) -> None:
        """Copies rows [lo, hi) of this rank's tensor into the same rows of every peer's. Peer (rank + s) is served in
        slot s, so that in every slot each GPU receives from exactly one sender. The copies go to `streams` in turn
        (the current stream if none is given): copies on different streams run on different copy engines at once,
        which one stream's queue of copies, each to another peer, does not."""
        import ctypes

        if not streams:
            streams = [torch.cuda.current_stream(self.tensor.device)]
        off, nbytes = lo * self.row_bytes, (hi - lo) * self.row_bytes
        for step in range(1, self.world):
            peer = (self.rank + step) % self.world
            stream = ctypes.c_void_p(streams[(step - 1) % len(streams)].cuda_stream)
            self.check("tc_peer_copy", self.lib.tc_peer_copy(ctypes.c_void_p(self.ptrs[peer] + off),
                                                             ctypes.c_void_p(self.ptrs[self.rank] + off), nbytes, stream))

    def fence(self) -> None:
        """Orders the current stream after every rank's pushes that precede ITS fence: a one-element all-reduce,
        which no rank's stream passes before all ranks' streams have reached it."""
        dist.all_reduce(self.flag, group=self.group)

    def close(self) -> None:
        import ctypes

        for r, raw in enumerate(self.bases):
            if raw is None:
                continue
            entry = _OPENED_PEER_ALLOCATIONS.get(raw)
            if entry is not None:
                entry[1] -= 1
                if entry[1] <= 0:
                    self.lib.tc_peer_close(ctypes.c_void_p(entry[0]))
                    del _OPENED_PEER_ALLOCATIONS[raw]
            self.bases[r] = None


class OverlappedAssembly:
    """Computes this rank's unit range of a sharded output in `blocks` pieces and, as soon as a piece is finished, pushes
    it into every other rank's copy of the output through peer windows (copy engines over NVLink), so that the
    assembly of the full output on every rank runs beside the computation of the later pieces instead of after it.
    `full` holds one unit per index of its first dimension (GEMM rows, (batch, head) pairs, ...), is contiguous and
    must be the same tensor on every call (the windows are opened once). Ranges are the balanced contiguous ones of
    aligned_shard_range; they need not be equal."""

    def __init__(self, blocks: int = 4, copy_streams: int = 1):
        # one copy stream: with the (rank + s) schedule every GPU then receives from one sender at a time, which
        # measured fastest on eight GPUs (2.00 ms for the 16384^3 GEMM against 2.22 / 2.88 ms with 7 / 4 streams).
        # Every peer copy costs about 34 us on top of its bytes, so on eight GPUs fewer blocks win (two: 1.89 ms,
        # four: 2.00, eight: 2.33), while on two or four, where the step is compute-bound, four or eight do.
        self.blocks = max(1, blocks)
        self.copy_streams = max(1, copy_streams)
        self.windows = None
        self.pushers = None

    def __call__(self, full: torch.Tensor, compute: Callable[[int, int], None], align: int = 1, group=None) -> Tuple[int, int]:
        total = full.shape[0]
        if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
            compute(0, total)
            return 0, total
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        start, stop = aligned_shard_range(total, world, rank, align)
        if self.windows is None or self.windows.key != (full.data_ptr(), tuple(full.shape)):
            if self.windows is not None:
                self.windows.close()
            self.windows = PeerWindows(full, group)
        if self.pushers is None:
            self.pushers = [torch.cuda.Stream(device=full.device) for _ in range(min(self.copy_streams, world - 1))]
        main = torch.cuda.current_stream(full.device)
        # piece boundaries: whole multiples of `align`, as even as they come
        units = (stop - start + align - 1) // align
        cuts = [start + min(stop - start, (units * j // self.blocks) * align) for j in range(self.blocks + 1)]
        for lo, hi in zip(cuts, cuts[1:]):
            if hi <= lo:
                continue
            compute(lo, hi)
            done = torch.cuda.Event()
            done.record(main)
            for s in self.pushers:
                s.wait_event(done)
            self.windows.push_rows(lo, hi, self.pushers)
        for s in self.pushers:
            main.wait_stream(s)
        self.windows.fence()    # every rank's pieces have arrived here once this completes
        return start, stop


def overlapped_flash_attn(assembly: OverlappedAssembly, q, k, v, o, scale=None, group=None) -> Tuple[int, int]:
    """sharded_flash_attn with O assembled on every rank while later (batch, head) groups are still computed."""
    from . import ops

    b, h = q.shape[:2]
    qf, kf, vf, of = (t.view(1, b * h, *t.shape[2:]) for t in (q, k, v, o))

    def compute(lo: int, hi: int) -> None:
        ops.flash_attn(qf[:, lo:hi], kf[:, lo:hi], vf[:, lo:hi], of[:, lo:hi], scale=scale)

    return assembly(of[0], compute, group=group)


class OverlappedGemm:
    """c = a @ b.T with the rows of a (and c) split across ranks and C assembled on every rank WHILE it is computed:
    a rank's slab is cut into row blocks, each block's GEMM runs on the caller's stream on `max_sms` SMs, and as soon
    as a block is finished it is exchanged with the other ranks from a side stream, so that the transfer of block j
    runs beside the GEMM of block j + 1 on the SMs the GEMM leaves free. Without a process group this is a plain
    GEMM. Slabs must be equal and divisible into `blocks` blocks of whole 128-row tiles; otherwise the gather
    follows the compute (all_gather_slabs)."""

    def __init__(self, blocks: int = 4, max_sms: int = 0, transport: str = "nccl", copy_streams: int = 1):
        """transport "nccl": grouped send / receive per block (needs SMs: give the GEMM a budget with max_sms);
        "copy_engine": every rank pushes its finished block into the other ranks' C through CUDA IPC windows
        (PeerWindows), which takes no SM, so the GEMM keeps them all; C must then be the same tensor on every call."""
        if transport not in ("nccl", "copy_engine"):
            raise ValueError("transport must be 'nccl' or 'copy_engine'")
        self.blocks = blocks
        self.max_sms = max_sms
        self.transport = transport
        self.side = None
        self.copy_streams = max(1, copy_streams)
        self.assembly = None

    def __call__(self, a: torch.Tensor, b: torch.Tensor, c: torch.Tensor, gather: bool = True, group=None) -> Tuple[int, int]:
        from . import ops

        if not (dist.is_available() and dist.is_initialized()):
            ops.gemm(a, b, c)
            return 0, a.shape[0]
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        m = a.shape[0]
        ranges = [aligned_shard_range(m, world, r, 128) for r in range(world)]
        start, stop = ranges[rank]
        rows = stop - start
        equal = len({hi - lo for lo, hi in ranges}) == 1
        if not gather or world == 1 or not equal or rows % (self.blocks * 128) != 0:
            if rows > 0:
                ops.gemm(a[start:stop], b, c[start:stop])
            if gather:
                all_gather_slabs(c, world, rank, ranges, group)
            return start, stop
        if self.side is None:
            self.side = torch.cuda.Stream(device=c.device)
        main = torch.cuda.current_stream(c.device)
        per = rows // self.blocks
        if self.transport == "copy_engine":
            if self.assembly is None:
                self.assembly = OverlappedAssembly(self.blocks, self.copy_streams)
            return self.assembly(c, lambda lo, hi: ops.gemm(a[lo:hi], b, c[lo:hi], max_sms=self.max_sms), align=128, group=group)
        works = []
        for j in range(self.blocks):
            lo, hi = j * per, (j + 1) * per
            # the last block has nothing to hide behind: give it every SM
            ops.gemm(a[start + lo:start + hi], b, c[start + lo:start + hi], max_sms=self.max_sms if j + 1 < self.blocks else 0)
            done = torch.cuda.Event()
            done.record(main)
            self.side.wait_event(done)
            with torch.cuda.stream(self.side):
                works += exchange_row_block(c, ranges, lo, hi, group)
        for w in works:
            w.wait()            # the caller's stream waits for the transfers
        main.wait_stream(self.side)
        return start, stop


class HostGemmPipeline:
    """The sharded GEMM for callers whose operands live in HOST memory, one rank per GPU:

        this rank's rows of A   host -> device in row blocks (its own slab only),
        B                       each rank uploads 1/world of it and the ranks all-gather the slices over NVLink,
                                so that B crosses each host link once in total instead of once per rank,
        C                       this rank's slab, device -> host block by block as the products finish.

    Uploads, products and downloads run on three streams and overlap. Buffers are allocated once (device staging
    for the A slab, B and the C slab); host tensors should be pinned. Without a process group the one rank uploads
    all of B."""

    def __init__(self, rows: int, n: int, k: int, device, blocks: int = 4, group=None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if n % self.world != 0 or rows % blocks != 0:
            raise ValueError("N must divide by the world size and the slab by the block count")
        self.rows, self.n, self.k, self.blocks = rows, n, k, blocks
        self.d_a = torch.empty(rows, k, dtype=torch.float16, device=device)
        self.d_b = torch.empty(n, k, dtype=torch.float16, device=device)
        self.d_c = torch.empty(rows, n, dtype=torch.float32, device=device)
        self.s_in = torch.cuda.Stream(device=device)
        self.s_out = torch.cuda.Stream(device=device)

    def b_slice(self) -> Tuple[int, int]:
        per = self.n // self.world
        return self.rank * per, (self.rank + 1) * per

    def __call__(self, h_a_slab: torch.Tensor, h_b_slice: torch.Tensor, h_c_slab: torch.Tensor) -> None:
        from . import ops

        main = torch.cuda.current_stream(self.d_a.device)
        lo, hi = self.b_slice()
        self.s_in.wait_stream(main)
        self.s_out.wait_stream(main)
        with torch.cuda.stream(self.s_in):
            self.d_b[lo:hi].copy_(h_b_slice, non_blocking=True)
            b_up = torch.cuda.Event()
            b_up.record(self.s_in)
            per = self.rows // self.blocks
            a_up = []
            for i in range(self.blocks):
                self.d_a[i * per:(i + 1) * per].copy_(h_a_slab[i * per:(i + 1) * per], non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(self.s_in)
                a_up.append(ev)
        main.wait_event(b_up)
        if self.world > 1:
            dist.all_gather_into_tensor(self.d_b, self.d_b[lo:hi], group=self.group)
        for i in range(self.blocks):
            main.wait_event(a_up[i])
            ops.gemm(self.d_a[i * per:(i + 1) * per], self.d_b, self.d_c[i * per:(i + 1) * per])
            done = torch.cuda.Event()
            done.record(main)
            self.s_out.wait_event(done)
            with torch.cuda.stream(self.s_out):
                h_c_slab[i * per:(i + 1) * per].copy_(self.d_c[i * per:(i + 1) * per], non_blocking=True)
        main.wait_stream(self.s_out)
