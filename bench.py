#!/usr/bin/env python
"""Benchmark of the tile-kernel path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

Prints ONE JSON line (rank 0). The headline workload is the fp16 GEMM 8192^3 (fp32 accumulate and
output), the configuration the TFLOP/s metric and its target are quoted on; a "step" is one GEMM.
With N > 1 (launched under torchrun, one rank per GPU) every rank computes its own 8192-row slab
of a GEMM with M = 8192*N against the replicated B: weak scaling, no collective on the data path;
the optional all-gather that assembles C on every rank is timed separately and reported under
"assemble". `value` counts the work of all ranks over the max-over-ranks device time.

Other workloads of the path (B2B GEMM, attention forward, LSTM chain, scatter_nd, GEMM sizes) are
timed briefly at N = 1 and reported under "others"; `--workload` makes any of them the headline.
`--impl reference` times the reference's CPU path for the same workload (the torch fp32 computation
its own tests use as ground truth) on the host cores, on a bounded sample.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

NOMINAL_TFLOPS = 2250.0
NOMINAL_HBM_GBS = 8000.0
FALLBACK_TFLOPS = 1590.0
FALLBACK_HBM_GBS = 6650.0
SEED = 1234  # the seed of the reference's Python tests

# DRAM bytes (read + write) per launch of the dominant kernel, from the ncu captures summarised under
# profiles/ (file named per entry). None where no capture exists.
NCU_TRAFFIC_BYTES: dict[str, int | None] = {
    "gemm8192": 1_079_000_000,   # profiles/gemm_8192_ncu.md
    "scatter": 1_387_700_000,    # profiles/scatter_nd_c5_ncu.md
    "fa": 2_128_600_000,         # profiles/flash_attn_c3_ncu.md
    "b2b": 12_680_000,           # profiles/b2b_gemm_c2_ncu.md (4.29 MB read in the kernel + 8.39 MB result written back)
}


def measured_peaks() -> dict:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"tflops": float(d["bf16_tflops"]), "tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                "hbm_gbs": float(d["hbm_gbs"]), "source": "measured"}
    return {"tflops": FALLBACK_TFLOPS, "tflops_sustained": 1400.0, "hbm_gbs": FALLBACK_HBM_GBS, "source": "fallback"}


# ----------------------------------------------------------------------------------------------------
# clocks
# ----------------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clock, power and throttle reasons of one GPU (read-only NVML queries) every few
    milliseconds while a timed region runs; falls back to `nvidia-smi -lms` if NVML cannot be loaded."""

    REASONS = {"hw_slowdown": 0x8, "sw_power_cap": 0x4, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40}
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.samples: list[tuple[float, int]] = []
        self.sm_max = None
        self.power: list[float] = []
        self._stop = threading.Event()
        self.thread = None
        self.proc = None
        self.lines: list[str] = []

    def _physical_index(self) -> int:
        vis = os.environ.get("CUDA_VISIBLE_DEVICES")
        if vis:
            ids = [x.strip() for x in vis.split(",") if x.strip()]
            if self.index < len(ids) and ids[self.index].isdigit():
                return int(ids[self.index])
        return self.index

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nvml = pynvml
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(self._physical_index())
            self.sm_max = float(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
            self.thread = threading.Thread(target=self._poll, daemon=True)
            self.thread.start()
            return
        except Exception:
            self.nvml = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100", "-i",
                 str(self._physical_index())], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _poll(self):
        n = self.nvml
        while not self._stop.is_set():
            try:
                mhz = float(n.nvmlDeviceGetClockInfo(self.handle, n.NVML_CLOCK_SM))
                try:
                    mask = int(n.nvmlDeviceGetCurrentClocksEventReasons(self.handle))
                except Exception:
                    mask = int(n.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle))
                self.samples.append((mhz, mask))
                if (len(self.samples) & 7) == 1:   # power is the slow query: every eighth round is enough
                    self.power.append(n.nvmlDeviceGetPowerUsage(self.handle) / 1000.0)
            except Exception:
                pass
            time.sleep(0.0005)

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if getattr(self, "nvml", None) is not None:
            self._stop.set()
            self.thread.join(timeout=2)
            reasons = sorted(name for name, bit in self.REASONS.items() if any(m & bit for _, m in self.samples))
            sm = [x for x, _ in self.samples]
            return {"sm_mhz": statistics.median(sm) if sm else None, "sm_min_mhz": min(sm) if sm else None,
                    "sm_max_mhz": self.sm_max, "power_w_max": round(max(self.power), 1) if self.power else None,
                    "samples": len(sm), "reasons": reasons, "source": "nvml"}
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["clock sampling unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                smax.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "samples": len(sm), "reasons": sorted(reasons), "source": "nvidia-smi"}


# ----------------------------------------------------------------------------------------------------
# workloads: each returns the tensors it needs and a step() that launches on the current stream
# ----------------------------------------------------------------------------------------------------
class Workload:
    name = ""
    metric = ""
    unit = "TFLOP/s"
    dtype = "f16"
    bound = "tensor"

    def units_per_step(self) -> float:  # FLOP (or bytes) per step on one rank
        raise NotImplementedError

    def setup(self, device, rank: int):
        raise NotImplementedError

    def step(self):
        raise NotImplementedError

    def launches_per_step(self) -> int:
        return 1

    def describe(self) -> dict:
        return {}

    # end-to-end leg: host buffers, copies inside the timed region
    def e2e_setup(self):
        raise NotImplementedError

    def e2e_step(self):
        raise NotImplementedError

    def e2e_bytes(self) -> tuple[int, int]:
        raise NotImplementedError

    # CPU leg (the reference's torch fp32 computation), bounded sample
    def cpu_sample(self):
        """Returns (callable, units_done_per_call, description)."""
        raise NotImplementedError


def rotation_sets(footprint_bytes: int) -> int:
    """How many copies of a workload's buffers make one pass over them exceed L2 (126 MB) with margin."""
    return 1 if footprint_bytes > 126e6 else int(-(-160e6 // footprint_bytes))


class GemmWorkload(Workload):
    def __init__(self, n: int):
        self.n = n
        self.name = f"gemm{n}"
        self.metric = f"fp16 GEMM {n}^3 TFLOP/s (fp32 accumulate, fp32 output)"

    def units_per_step(self):
        return 2.0 * self.n ** 3

    def footprint(self):
        return 2 * self.n * self.n * 2 + self.n * self.n * 4

    def setup(self, device, rank):
        n = self.n
        g = torch.Generator(device=device).manual_seed(SEED + rank)
        self.a = (torch.rand(n, n, generator=g, device=device) * 2 - 1).half()
        gb = torch.Generator(device=device).manual_seed(SEED)
        self.b = (torch.rand(n, n, generator=gb, device=device) * 2 - 1).half()
        self.c = torch.empty(n, n, device=device)
        # small problems: enough copies of the operands and outputs that one pass over them exceeds L2, used in
        # rotation, so that every step reads cold data while the code stays warm
        self.sets = [(self.a, self.b, self.c)]
        for _ in range(rotation_sets(self.footprint()) - 1):
            self.sets.append((self.a.clone(), self.b.clone(), torch.empty_like(self.c)))
        self.turn = 0

    def step(self):
        from tiledcuda_b200 import ops
        a, b, c = self.sets[self.turn]
        self.turn = (self.turn + 1) % len(self.sets)
        ops.gemm(a, b, c)

    def describe(self):
        n = self.n
        sets = rotation_sets(self.footprint())
        return {"M_per_gpu": n, "N": n, "K": n, "a": "row-major fp16", "b": "col-major fp16 ([N,K] rows)", "c": "fp32",
                "l2": "inputs+output larger than L2" if sets == 1 else
                      f"{sets} operand/output sets of {self.footprint() / 1e6:.1f} MB used in rotation (together larger than L2)",
                "flush_l2": False,
                # a step of a few microseconds: a CUDA graph of one pass over the sets replaces the Python call path
                **({"graph_steps": sets, "launch": f"CUDA graph of {sets} steps"} if n <= 2048 else {})}

    def e2e_setup(self):
        from tiledcuda_b200 import ops
        self.ha = self.a.cpu().pin_memory()
        self.hb = self.b.cpu().pin_memory()
        self.hc = torch.empty(self.n, self.n, dtype=torch.float32).pin_memory()
        self.ws = torch.empty(ops.gemm_host_workspace_bytes(self.n, self.n, self.n), dtype=torch.uint8, device=self.a.device)

    def e2e_step(self):
        # the host-buffer entry point: uploads of A and B, the products and the download of C inside the call
        from tiledcuda_b200 import ops
        ops.gemm_host(self.ha, self.hb, self.hc, self.ws)

    def e2e_bytes(self):
        return 2 * self.n * self.n * 2, self.n * self.n * 4

    def cpu_sample(self):
        n = self.n
        rows = min(n, max(128, int(2.0e11 / (2.0 * n * n)) // 128 * 128))
        a = self.a[:rows].cpu() if hasattr(self, "a") else (torch.rand(rows, n) * 2 - 1).half()
        b = self.b.cpu() if hasattr(self, "b") else (torch.rand(n, n) * 2 - 1).half()
        a32, b32 = a.float(), b.float()

        def run():
            return a32 @ b32.t()

        return run, 2.0 * rows * n * n, f"{rows} of {n} rows of A against the full B (fp32 torch matmul), scaled by FLOPs"


class B2bWorkload(Workload):
    name = "b2b"
    metric = "fp16 back-to-back GEMM 16384x128x128x128 TFLOP/s"
    bound = "hbm"

    def units_per_step(self):
        return 2.0 * 16384 * 128 * 128 * 2

    def bytes_per_step(self):
        return 2 * (16384 * 128 + 128 * 128 + 128 * 128) + 4 * 16384 * 128

    def setup(self, device, rank):
        g = torch.Generator(device=device).manual_seed(SEED + rank)
        self.a = (torch.randn(16384, 128, generator=g, device=device) * 0.1).half()
        self.b = (torch.randn(128, 128, generator=g, device=device) * 0.1).half()
        self.d = (torch.randn(128, 128, generator=g, device=device) * 0.1).half()
        self.e = torch.empty(16384, 128, device=device)
        self.sets = [(self.a, self.b, self.d, self.e)]
        for _ in range(rotation_sets(self.bytes_per_step()) - 1):
            self.sets.append((self.a.clone(), self.b.clone(), self.d.clone(), torch.empty_like(self.e)))
        self.turn = 0

    def step(self):
        from tiledcuda_b200 import ops
        a, b, d, e = self.sets[self.turn]
        self.turn = (self.turn + 1) % len(self.sets)
        ops.back2back_gemm(a, b, d, e)

    def describe(self):
        sets = rotation_sets(self.bytes_per_step())
        return {"M": 16384, "N": 128, "K": 128, "P": 128,
                "l2": f"{sets} operand/output sets of {self.bytes_per_step() / 1e6:.1f} MB used in rotation (together larger than L2)",
                "flush_l2": False, "graph_steps": sets, "launch": f"CUDA graph of {sets} steps"}

    def cpu_sample(self):
        a, b, d = self.a.cpu().float(), self.b.cpu().float(), self.d.cpu().float()

        def run():
            return ((a @ b.t()).half().float()) @ d.t()

        return run, self.units_per_step(), "full problem (fp32 torch, intermediate rounded to fp16)"


class AttentionWorkload(Workload):
    name = "fa"
    metric = "FlashAttention-2 forward b16 h32 s4096 d128 TFLOP/s"

    def __init__(self, batch=16, heads=32, seq=4096, dim=128):
        self.batch, self.heads, self.seq, self.dim = batch, heads, seq, dim

    def units_per_step(self):
        return 4.0 * self.batch * self.heads * self.seq * self.seq * self.dim

    def setup(self, device, rank):
        g = torch.Generator(device=device).manual_seed(SEED + rank)
        shape = (self.batch, self.heads, self.seq, self.dim)
        self.q = torch.randn(shape, generator=g, device=device, dtype=torch.float16)
        self.k = torch.randn(shape, generator=g, device=device, dtype=torch.float16)
        self.v = torch.randn(shape, generator=g, device=device, dtype=torch.float16)
        self.o = torch.empty_like(self.q)

    def step(self):
        from tiledcuda_b200 import ops
        ops.flash_attn(self.q, self.k, self.v, self.o)

    def cpu_sample(self):
        heads = 4
        q, k, v = (t[0, :heads].cpu().float() for t in (self.q, self.k, self.v))
        scale = 1.0 / math.sqrt(self.dim)

        def run():
            return torch.softmax((q @ k.transpose(-1, -2)) * scale, dim=-1) @ v

        return run, 4.0 * heads * self.seq * self.seq * self.dim, f"1 batch x {heads} heads of {self.batch}x{self.heads} (fp32 torch), scaled by FLOPs"


class LstmWorkload(Workload):
    name = "lstm"
    metric = "LSTM chain b256 i1024 h1024 x64 steps TFLOP/s"
    steps, batch, inp, hidden = 64, 256, 1024, 1024

    def units_per_step(self):
        return 2.0 * 4 * self.hidden * (self.inp + self.hidden) * self.batch * self.steps

    def setup(self, device, rank):
        g = torch.Generator(device=device).manual_seed(SEED + rank)
        self.w = (torch.randn(4 * self.hidden, self.inp, generator=g, device=device) * 0.02).half()
        self.u = (torch.randn(4 * self.hidden, self.hidden, generator=g, device=device) * 0.02).half()
        self.x = torch.randn(self.steps, self.batch, self.inp, generator=g, device=device).half()
        self.h0 = torch.zeros(self.batch, self.hidden, dtype=torch.float16, device=device)
        self.c0 = torch.zeros(self.batch, self.hidden, device=device)
        self.h_all = torch.empty(self.steps, self.batch, self.hidden, dtype=torch.float16, device=device)
        self.c_t = torch.empty(self.batch, self.hidden, device=device)
        if device.type == "cuda":
            from tiledcuda_b200 import ops
            self.ws = torch.empty(ops.lstm_chain_workspace_bytes(self.steps, self.batch, self.hidden) // 4, device=device)

    def step(self):
        from tiledcuda_b200 import ops
        ops.lstm_chain(self.w, self.u, None, self.x, self.h0, self.c0, self.h_all, self.c_t, workspace=self.ws)

    def launches_per_step(self):
        return self.steps + 1  # one GEMM for the input projections of all steps, then one launch per step

    def describe(self):
        # 65 launches of a few microseconds each: replayed from a CUDA graph so that the host's launch path is
        # not what is timed. Weights, inputs and the 268 MB projection workspace together exceed L2.
        return {"steps_per_chain": self.steps, "batch": self.batch, "input": self.inp, "hidden": self.hidden,
                "l2": "weights + inputs + workspace larger than L2", "flush_l2": False,
                "graph_steps": 1, "launch": "CUDA graph of one chain (65 kernels)"}

    def cpu_sample(self):
        from oracle import oracle
        w, u, x, h0, c0 = (t.cpu() for t in (self.w, self.u, self.x, self.h0, self.c0))

        def run():
            return oracle.lstm_chain(w, u, None, x, h0, c0)

        return run, self.units_per_step(), "full 64-step chain (fp32 torch)"


class ScatterWorkload(Workload):
    name = "scatter"
    metric = "scatter_nd 2^24 rows into [2^26, 8] fp16 GB/s"
    unit = "GB/s"
    dtype = "i32 index / 16-byte rows"
    bound = "hbm"
    rows, width, n = 1 << 26, 8, 1 << 24
    rotate = 4  # update / index sets rotated so that no step finds its inputs in L2

    def units_per_step(self):
        return float(self.n * (4 + 16 + 16))

    def setup(self, device, rank):
        g = torch.Generator(device=device).manual_seed(SEED + rank)
        self.table = torch.randn(self.rows, self.width, generator=g, device=device, dtype=torch.float16)
        self.idx = [torch.randperm(self.rows, generator=g, device=device)[: self.n].to(torch.int32).view(-1, 1).contiguous()
                    for _ in range(self.rotate)]
        self.upd = [torch.randn(self.n, self.width, generator=g, device=device, dtype=torch.float16) for _ in range(self.rotate)]
        self.i = 0

    def step(self):
        from tiledcuda_b200 import ops
        j = self.i % self.rotate
        self.i += 1
        ops.scatter_nd(self.table, self.idx[j], self.upd[j])

    def describe(self):
        return {"table": "[2^26, 8] fp16", "updates": "2^24 unique rows", "l2": f"{self.rotate} rotating index/update sets (320 MB each) larger than L2"}

    def cpu_sample(self):
        table = self.table.cpu()
        idx = self.idx[0].cpu().view(-1).long()
        upd = self.upd[0].cpu()

        def run():
            table[idx] = upd
            return table

        return run, self.units_per_step(), "full problem (torch index assignment)"


def make_workload(name: str) -> Workload:
    if name.startswith("gemm"):
        return GemmWorkload(int(name[4:]))
    return {"b2b": B2bWorkload, "fa": AttentionWorkload, "lstm": LstmWorkload, "scatter": ScatterWorkload}[name]()


# ----------------------------------------------------------------------------------------------------
# timing
# ----------------------------------------------------------------------------------------------------
def flush_l2(device, scratch=[None]):
    if scratch[0] is None:
        scratch[0] = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    scratch[0].fill_(1)


def time_steps(fn, steps: int, warmup: int, barrier, flush=False, device=None, on_timed_start=None, graph: int = 0) -> float:
    """Milliseconds per step on the device, CUDA events on the launching stream, barrier + sync on both sides.
    graph = G > 0: G consecutive steps are captured into one CUDA graph and the timed region replays it
    ceil(steps / G) times (for kernels of a few microseconds, which the Python call path cannot feed fast enough)."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    barrier()
    if graph > 0:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                for _ in range(graph):
                    fn()
        torch.cuda.current_stream().wait_stream(side)
        g.replay()
        torch.cuda.synchronize()
        replays = -(-steps // graph)
        if on_timed_start is not None:
            on_timed_start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(replays):
            g.replay()
        e1.record()
        torch.cuda.synchronize()
        barrier()
        return e0.elapsed_time(e1) / (replays * graph)
    if on_timed_start is not None:
        on_timed_start()
    if flush:
        total = 0.0
        for _ in range(steps):
            flush_l2(device)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            e1.synchronize()
            total += e0.elapsed_time(e1)
        barrier()
        return total / steps
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    barrier()
    return e0.elapsed_time(e1) / steps


def best_of_steps(fn, reps: int, barrier) -> float:
    """Milliseconds of the fastest of `reps` steps, each timed alone after a pause in which the GPU idles: the
    way the burst GEMM peak in MEASURED_PEAKS.json was taken (best of 10), before the power cap lowers the clock."""
    best = float("inf")
    for _ in range(reps):
        torch.cuda.synchronize()
        time.sleep(0.05)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        e1.synchronize()
        best = min(best, e0.elapsed_time(e1))
    barrier()
    return best


def roofline(w: Workload, ms: float, peaks: dict, burst_ms: float | None = None) -> dict:
    if w.bound == "tensor":
        achieved = w.units_per_step() / w.launches_per_step() / (ms / w.launches_per_step() * 1e-3) / 1e12
        peak, unit, nominal = peaks["tflops"], "TFLOP/s", NOMINAL_TFLOPS
        if burst_ms is not None:
            # `achieved` comes from the back-to-back loop (power-capped clocks) and is set against the burst peak,
            # the stricter of the two denominators; the like-for-like pairs are loop vs sustained and burst vs burst.
            burst = w.units_per_step() / (burst_ms * 1e-3) / 1e12
            return {"bound": w.bound, "achieved": round(achieved, 2), "peak": peak, "unit": unit, "frac": round(achieved / peak, 4),
                    "peak_source": peaks["source"], "frac_of_nominal": round(achieved / nominal, 4),
                    "peak_sustained": peaks["tflops_sustained"], "frac_of_sustained": round(achieved / peaks["tflops_sustained"], 4),
                    "achieved_burst": round(burst, 2), "frac_burst": round(burst / peak, 4),
                    "burst_how": "fastest of 10 single steps, each after a 50 ms idle pause",
                    "traffic": NCU_TRAFFIC_BYTES.get(w.name)}
    else:
        nbytes = w.bytes_per_step() if hasattr(w, "bytes_per_step") else w.units_per_step()
        achieved = nbytes / (ms * 1e-3) / 1e9
        peak, unit, nominal = peaks["hbm_gbs"], "GB/s", NOMINAL_HBM_GBS
    return {"bound": w.bound, "achieved": round(achieved, 2), "peak": peak, "unit": unit, "frac": round(achieved / peak, 4),
            "peak_source": peaks["source"], "frac_of_nominal": round(achieved / nominal, 4), "traffic": NCU_TRAFFIC_BYTES.get(w.name)}


def cpu_baseline(w: Workload, reps: int = 2) -> dict:
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    run, units, sample = w.cpu_sample()
    run()
    best = float("inf")
    for _ in range(reps):
        t0 = time.perf_counter()
        run()
        best = min(best, time.perf_counter() - t0)
    scale = 1e12 if w.unit == "TFLOP/s" else 1e9
    return {"value": round(units / best / scale, 4), "unit": w.unit, "cores": threads, "kind": "port",
            "sample": sample, "seconds_per_sample": round(best, 4)}


def run_reference_arm(args, w: Workload, rank: int) -> int:
    """The reference's CPU path (its tests' torch fp32 computation) on the host cores; rank 0 only."""
    if rank != 0:
        return 0
    # inputs on the host: build the workload's CPU sample without touching a GPU
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    run, units, sample = _cpu_only_sample(w)
    for _ in range(max(1, min(args.warmup, 2))):
        run()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        run()
    dt = (time.perf_counter() - t0) / args.steps
    scale = 1e12 if w.unit == "TFLOP/s" else 1e9
    value = round(units / dt / scale, 4)
    ref_cuda = reference_cuda_gemm()
    line = {
        "impl": "reference", "metric": w.metric, "value": value, "unit": w.unit, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(dt * 1e3, 3), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32 (torch CPU reference of the fp16 op)", "data": "synthetic",
        "config": {"workload": w.name, **w.describe()},
        "cpu_baseline": {"value": value, "unit": w.unit, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": w.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    if ref_cuda is not None:
        line["reference_cuda_kernel"] = ref_cuda
    print(json.dumps(line), flush=True)
    return 0


def reference_cuda_gemm() -> dict | None:
    """The reference's own CUDA GEMM example (4096^3, its native size; sm_80-style mma.sync kernel compiled
    unmodified for sm_100a into oracle/_ref/ by oracle/ref_build/Makefile), run once if it was built and a
    GPU is present. It prints `cuBLAS  TiledCUDA  Ratio` in milliseconds after checking itself against cuBLAS."""
    exe = ROOT / "oracle" / "_ref" / "ref_gemm_4096"
    if not exe.exists() or not torch.cuda.is_available():
        return None
    try:
        res = subprocess.run([str(exe)], capture_output=True, text=True, timeout=120, cwd=str(exe.parent))
    except (OSError, subprocess.TimeoutExpired) as e:
        return {"unavailable": f"{type(e).__name__}"}
    lines = [l for l in res.stdout.strip().splitlines() if l.strip()]
    try:
        cublas_ms, ref_ms, _ = (float(x) for x in lines[-1].split())
    except (ValueError, IndexError):
        return {"unavailable": f"exit {res.returncode}: {(res.stdout + res.stderr)[-200:]}"}
    flops = 2.0 * 4096 ** 3
    return {"workload": "fp16 GEMM 4096^3 (reference example 02_gemm_all_mem, CTA tile 64x256x32)", "self_check": "Test passed." in res.stdout,
            "ms": ref_ms, "tflops": round(flops / ref_ms / 1e9, 1), "cublas_hgemm_ms": cublas_ms,
            "cublas_hgemm_tflops": round(flops / cublas_ms / 1e9, 1)}


def _cpu_only_sample(w: Workload):
    """CPU sample with inputs generated on the host (no GPU involved)."""
    if isinstance(w, GemmWorkload):
        n = w.n
        rows = min(n, max(128, int(2.0e11 / (2.0 * n * n)) // 128 * 128))
        g = torch.Generator().manual_seed(SEED)
        a32 = (torch.rand(rows, n, generator=g) * 2 - 1).half().float()
        b32 = (torch.rand(n, n, generator=g) * 2 - 1).half().float()
        return (lambda: a32 @ b32.t()), 2.0 * rows * n * n, f"{rows} of {n} rows of A against the full B (fp32 torch matmul), scaled by FLOPs"
    w.setup(torch.device("cpu"), 0)
    return w.cpu_sample()


# ----------------------------------------------------------------------------------------------------
# main
# ----------------------------------------------------------------------------------------------------
def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="gemm8192",
                    help="gemm<N> | b2b | fa | lstm | scatter (default gemm8192)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-others", action="store_true", help="skip the brief timing of the other workloads")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end leg")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    w = make_workload(args.workload)

    if args.impl == "reference":
        return run_reference_arm(args, w, rank)

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the kernels are sm_100a only and there is no CPU path")
    from tiledcuda_b200 import _lib
    _lib.load()  # fail loudly if the native library is missing

    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    distributed = world > 1
    if distributed:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)
        barrier = lambda: (dist.barrier(), torch.cuda.synchronize())
    else:
        barrier = lambda: torch.cuda.synchronize()

    peaks = measured_peaks()
    w.setup(device, rank)
    desc = w.describe()

    sampler = ClockSampler(local_rank)
    ms = time_steps(w.step, args.steps, args.warmup, barrier, flush=bool(desc.get("flush_l2")), device=device,
                    on_timed_start=sampler.start, graph=int(desc.get("graph_steps", 0)))
    clocks = sampler.stop()
    burst_ms = best_of_steps(w.step, 10, barrier) if (w.bound == "tensor" and w.launches_per_step() == 1) else None
    status = _lib.device_status()

    ms_t = torch.tensor([ms], device=device, dtype=torch.float64)
    if distributed:
        dist.all_reduce(ms_t, op=dist.ReduceOp.MAX)
    ms_max = ms_t.item()
    scale = 1e12 if w.unit == "TFLOP/s" else 1e9
    value = w.units_per_step() * world / (ms_max * 1e-3) / scale

    # assemble leg (multi-GPU): all-gather of the output slabs, timed on its own
    assemble = None
    if distributed and isinstance(w, GemmWorkload):
        full = torch.empty(world * w.n, w.n, device=device)
        full[rank * w.n:(rank + 1) * w.n].copy_(w.c)

        def gather():
            dist.all_gather_into_tensor(full, full[rank * w.n:(rank + 1) * w.n])

        g_ms = time_steps(gather, max(3, args.steps // 4), 2, barrier)
        g_t = torch.tensor([g_ms], device=device, dtype=torch.float64)
        dist.all_reduce(g_t, op=dist.ReduceOp.MAX)
        assemble = {"collective": "nccl all_gather of C (fp32)", "ms": round(g_t.item(), 4),
                    "bytes_received_per_gpu": (world - 1) * w.n * w.n * 4,
                    "bus_gbs": round((world - 1) * w.n * w.n * 4 / (g_t.item() * 1e-3) / 1e9, 1)}
        del full

    # end-to-end leg: host buffers, copies inside the timed region
    e2e = None
    if isinstance(w, GemmWorkload) and not args.no_e2e:
        w.e2e_setup()
        e_steps = max(3, min(args.steps, 10))
        e_ms = time_steps(w.e2e_step, e_steps, 3, barrier)
        e_t = torch.tensor([e_ms], device=device, dtype=torch.float64)
        if distributed:
            dist.all_reduce(e_t, op=dist.ReduceOp.MAX)
        h2d, d2h = w.e2e_bytes()
        e2e = {"value": round(w.units_per_step() * world / (e_t.item() * 1e-3) / scale, 3), "unit": w.unit,
               "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": round(e_t.item(), 3), "steps": e_steps}

    line = {
        "metric": w.metric, "value": round(value, 2), "unit": w.unit, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms_max, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": w.dtype, "data": "synthetic",
        "config": {"workload": w.name, **desc, "parallelism": f"dp{world} (row slabs, no data-path collective)"},
        "roofline": roofline(w, ms, peaks, burst_ms),
        "clocks": clocks,
        "gpu_launches": (-(-args.steps // int(desc["graph_steps"])) * int(desc["graph_steps"]) if desc.get("graph_steps")
                         else args.steps) * w.launches_per_step(),
        "device_status": status,
    }
    if e2e is not None:
        line["e2e"] = e2e
    if assemble is not None:
        line["assemble"] = assemble

    if rank == 0 and world == 1:
        if not args.no_cpu:
            line["cpu_baseline"] = cpu_baseline(w)
        if not args.no_others:
            others = {}
            del w
            torch.cuda.empty_cache()
            # Light workloads first and half a second of idle GPU before each: a kernel that ran into the power cap
            # leaves the clock governor throttling for a while, and the workload timed right behind it pays for that
            # (attention right behind the 16384^3 GEMM: 5.8 ms against 4.1 ms from idle).
            for name in ("gemm1024", "gemm2048", "b2b", "lstm", "scatter", "fa", "gemm4096", "gemm16384"):
                if name == args.workload:
                    continue
                ow = make_workload(name)
                ow.setup(device, 0)
                od = ow.describe()
                torch.cuda.synchronize()
                time.sleep(0.5)
                # short kernels need many launches for the host to stay ahead of the device
                steps = {"gemm16384": 5, "gemm1024": 300, "gemm2048": 200, "b2b": 300}.get(name, 10)
                ograph = int(od.get("graph_steps", 0))
                oms = time_steps(ow.step, steps, 3, barrier, flush=bool(od.get("flush_l2")), device=device, graph=ograph)
                oscale = 1e12 if ow.unit == "TFLOP/s" else 1e9
                others[name] = {"metric": ow.metric, "value": round(ow.units_per_step() / (oms * 1e-3) / oscale, 2), "unit": ow.unit,
                                "ms_per_step": round(oms, 4), "roofline": roofline(ow, oms, peaks), "launches_per_step": ow.launches_per_step()}
                del ow
                torch.cuda.empty_cache()
            others["device_status"] = _lib.device_status()
            line["others"] = others

    if distributed:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        print(json.dumps(line), flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
