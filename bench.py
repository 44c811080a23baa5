#!/usr/bin/env python
"""Benchmark of the tile-kernel path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

Prints ONE JSON line (rank 0). The headline workload is the fp16 GEMM 8192^3 (fp32 accumulate and
output), the configuration the TFLOP/s metric and its target are quoted on; a "step" is one GEMM.

What the line carries for the headline workload:
  value / ms_per_step   K steps back to back, inputs resident in HBM, CUDA events, max over ranks
  roofline              achieved vs the measured peak; a burst figure (fastest of 10 isolated launches) beside it
  sustained             the same step looped for >= 2 s of device time with SM clock, power and throttle reasons
                        sampled across the whole loop; its fraction is taken against the SUSTAINED peak only
  parity                max-abs / relative-Frobenius error (scatter: bit_exact) of one checked launch against
                        the CPU reference computation, outside every timed region
  e2e                   the same work through the host-buffer call: operands start in pinned host memory and the
                        result returns to it inside the timed region
  cpu_baseline          the reference's CPU path (the torch fp32 computation its tests use as ground truth)
                        timed on the host cores on a bounded sample
The other workloads of the path (GEMM sizes, B2B GEMM, attention forward, LSTM chain, scatter_nd) are timed
at N = 1 under "others", each with its own roofline, clocks, parity and cpu_baseline.

With N > 1 (torchrun, one rank per GPU) everything goes through tiledcuda_b200/shard.py. `value` is weak
scaling: every rank computes its own 8192-row slab of a GEMM with M = 8192 N against the replicated B, no
collective on the data path. Beside it:
  strong   GEMM 16384^3 split along M with C assembled on every rank: compute alone, all-gather alone, and
           the overlapped form (row blocks exchanged from a side stream while later blocks compute)
  others   attention over batch x heads, the LSTM chain over batch and owner-computes scatter_nd, sharded, with
           the single-GPU time of the same problem measured in the same run
  e2e      host operands: each rank uploads its A slab and 1/N of B, B is all-gathered over NVLink
`--impl reference` times the reference's CPU path for the same workload on the host cores (rank 0 only).
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
SUSTAINED_SECONDS = 2.0

# DRAM bytes (read + write) per launch of the dominant kernel, from the ncu captures summarised under
# profiles/ (file named per entry). None where no capture exists.
NCU_TRAFFIC_BYTES: dict[str, int | None] = {
    "gemm8192": 1_079_000_000,   # profiles/gemm_8192_ncu.md
    "scatter": 1_387_700_000,    # profiles/scatter_nd_c5_ncu.md
    "fa": 2_130_000_000,         # profiles/flash_attn_c3_ncu.md
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


def bind_to_gpu_numa_node(local_rank: int) -> str | None:
    """Restricts this PROCESS to the host cores NVML names as closest to its GPU (a read-only query of the GPU;
    the only thing changed is this process's own CPU affinity), so that the pinned host buffers of a multi-rank
    run are first touched on the GPU's own memory node and eight ranks do not funnel through one."""
    try:
        import pynvml
        pynvml.nvmlInit()
        vis = os.environ.get("CUDA_VISIBLE_DEVICES")
        idx = local_rank
        if vis:
            ids = [x.strip() for x in vis.split(",") if x.strip()]
            if local_rank < len(ids) and ids[local_rank].isdigit():
                idx = int(ids[local_rank])
        handle = pynvml.nvmlDeviceGetHandleByIndex(idx)
        words = (os.cpu_count() + 63) // 64
        mask = pynvml.nvmlDeviceGetCpuAffinity(handle, words)
        cpus = {w * 64 + b for w, m in enumerate(mask) for b in range(64) if (int(m) >> b) & 1}
        cpus &= os.sched_getaffinity(0)
        if cpus:
            os.sched_setaffinity(0, cpus)
            return f"{len(cpus)} cores near GPU {idx}"
    except Exception as e:   # affinity is an optimisation; the run is valid without it
        return f"unchanged ({type(e).__name__})"
    return None


# ----------------------------------------------------------------------------------------------------
# error metrics (reported, not asserted: the tests hold the tolerances)
# ----------------------------------------------------------------------------------------------------
def error_metrics(out: torch.Tensor, ref: torch.Tensor, what: str) -> dict:
    o, r = out.detach().cpu().double(), ref.detach().cpu().double()
    return {"max_abs_err": float((o - r).abs().max()), "rel_fro_err": float((o - r).norm() / max(r.norm().item(), 1e-30)),
            "checked": what, "against": "fp32 torch CPU computation on the same fp16 inputs"}


# ----------------------------------------------------------------------------------------------------
# workloads: tensors, a step() that launches on the current stream, the CPU reference of a bounded sample,
# and an end-to-end step whose operands start and end in pinned host memory
# ----------------------------------------------------------------------------------------------------
class Workload:
    name = ""
    metric = ""
    unit = "TFLOP/s"
    dtype = "f16"
    bound = "tensor"
    graph_steps = 0          # > 0: this many consecutive steps are replayed from one CUDA graph
    others_steps = 10        # steps of the brief timing under "others"

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

    # one checked launch + the CPU computation of the same sample: returns (cpu_run, units, description, compare)
    # where cpu_run() -> CPU result and compare(cpu_result) -> parity dict (launches the product op once)
    def cpu_reference(self):
        raise NotImplementedError

    # end-to-end leg: host buffers, copies inside the timed region. Default: every input is copied up from pinned
    # memory, the op runs, every output is copied back, all on the current stream.
    def e2e_tensors(self):
        """(inputs, outputs): device tensors the step reads / writes."""
        raise NotImplementedError

    def e2e_setup(self):
        ins, outs = self.e2e_tensors()
        self._e2e_in = [(t, t.cpu().pin_memory()) for t in ins]
        self._e2e_out = [(t, torch.empty(t.shape, dtype=t.dtype).pin_memory()) for t in outs]

    def e2e_step(self):
        for dev, host in self._e2e_in:
            dev.copy_(host, non_blocking=True)
        self.step()
        for dev, host in self._e2e_out:
            host.copy_(dev, non_blocking=True)

    def e2e_bytes(self) -> tuple[int, int]:
        ins, outs = self.e2e_tensors()
        return sum(t.numel() * t.element_size() for t in ins), sum(t.numel() * t.element_size() for t in outs)

    def e2e_how(self) -> str:
        return "inputs copied from pinned host memory, op, outputs copied back, on one stream"


def rotation_sets(footprint_bytes: int) -> int:
    """How many copies of a workload's buffers make one pass over them exceed L2 (126 MB) with margin."""
    return 1 if footprint_bytes > 126e6 else int(-(-160e6 // footprint_bytes))


def cpu_rows_for(n: int) -> int:
    """Rows of A in the CPU sample of an n^3 GEMM: about 2e11 FLOP of fp32 work, whole 128-row tiles."""
    return min(n, max(128, int(2.0e11 / (2.0 * n * n)) // 128 * 128))


class GemmWorkload(Workload):
    def __init__(self, n: int):
        self.n = n
        self.name = f"gemm{n}"
        self.metric = f"fp16 GEMM {n}^3 TFLOP/s (fp32 accumulate, fp32 output)"
        sets = rotation_sets(self.footprint())
        self.graph_steps = sets if n <= 2048 else 0
        self.others_steps = {16384: 5, 1024: 300, 2048: 200}.get(n, 10)

    def units_per_step(self):
        return 2.0 * self.n ** 3

    def footprint(self):
        return 2 * self.n * self.n * 2 + self.n * self.n * 4

    def setup(self, device, rank):
        n = self.n
        # B first, from the seed alone: every rank holds the same B; then this rank's own rows of A
        gb = torch.Generator(device=device).manual_seed(SEED)
        self.b = (torch.rand(n, n, generator=gb, device=device) * 2 - 1).half()
        g = torch.Generator(device=device).manual_seed(SEED + 7919 * (rank + 1))
        self.a = (torch.rand(n, n, generator=g, device=device) * 2 - 1).half()
        self.c = torch.empty(n, n, device=device)
        # small problems: enough copies of the operands and outputs that one pass over them exceeds L2, used in
        # rotation, so that every step reads cold data while the code stays warm
        self.sets = [(self.a, self.b, self.c)]
        for _ in range(rotation_sets(self.footprint()) - 1):
            self.sets.append((self.a.clone(), self.b.clone(), torch.empty_like(self.c)))
        self.turn = 0

    def step(self):
        from tiledcuda_b200 import ops, shard
        a, b, c = self.sets[self.turn]
        self.turn = (self.turn + 1) % len(self.sets)
        # this rank's slab [start, stop) of a GEMM with M = n * world; one rank: the whole problem
        world = torch.distributed.get_world_size() if torch.distributed.is_initialized() else 1
        shard.run_sharded(self.n * world, lambda start, stop: ops.gemm(a, b, c), align=128)

    def describe(self):
        n = self.n
        sets = rotation_sets(self.footprint())
        return {"M_per_gpu": n, "N": n, "K": n, "a": "row-major fp16", "b": "col-major fp16 ([N,K] rows)", "c": "fp32",
                "l2": "inputs+output larger than L2" if sets == 1 else
                      f"{sets} operand/output sets of {self.footprint() / 1e6:.1f} MB used in rotation (together larger than L2)",
                "flush_l2": False,
                # a step of a few microseconds: a CUDA graph of one pass over the sets replaces the Python call path
                **({"graph_steps": sets, "launch": f"CUDA graph of {sets} steps"} if self.graph_steps else {})}

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

    def e2e_how(self):
        return "tc_gemm_f16_f32_host: A and B uploaded, block products, C downloaded, pipelined over three streams"

    def cpu_reference(self):
        from tiledcuda_b200 import ops
        n, rows = self.n, cpu_rows_for(self.n)
        a32, b32 = self.a[:rows].cpu().float(), self.b.cpu().float()

        def run():
            return a32 @ b32.t()

        def compare(ref):
            self.c.fill_(float("nan"))
            ops.gemm(self.a, self.b, self.c)
            return error_metrics(self.c[:rows], ref, f"rows 0..{rows - 1} of C ({rows} x {n})")

        return run, 2.0 * rows * n * n, f"{rows} of {n} rows of A against the full B (fp32 torch matmul), scaled by FLOPs", compare


class B2bWorkload(Workload):
    name = "b2b"
    metric = "fp16 back-to-back GEMM 16384x128x128x128 TFLOP/s"
    bound = "hbm"
    others_steps = 300

    def __init__(self):
        self.graph_steps = rotation_sets(self.bytes_per_step())

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

    def e2e_tensors(self):
        return [self.a, self.b, self.d], [self.e]

    def e2e_step(self):
        from tiledcuda_b200 import ops
        for dev, host in self._e2e_in:
            dev.copy_(host, non_blocking=True)
        ops.back2back_gemm(self.a, self.b, self.d, self.e)
        for dev, host in self._e2e_out:
            host.copy_(dev, non_blocking=True)

    def cpu_reference(self):
        from tiledcuda_b200 import ops
        a, b, d = self.a.cpu().float(), self.b.cpu().float(), self.d.cpu().float()

        def run():
            return ((a @ b.t()).half().float()) @ d.t()

        def compare(ref):
            self.e.fill_(float("nan"))
            ops.back2back_gemm(self.a, self.b, self.d, self.e)
            return error_metrics(self.e, ref, "the whole result (16384 x 128)")

        return run, self.units_per_step(), "full problem (fp32 torch, intermediate rounded to fp16)", compare


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

    def describe(self):
        return {"batch": self.batch, "heads": self.heads, "seq": self.seq, "head_dim": self.dim, "causal": False,
                "l2": "Q, K, V, O (2.1 GB) larger than L2", "flush_l2": False}

    def e2e_tensors(self):
        return [self.q, self.k, self.v], [self.o]

    def cpu_reference(self):
        heads = 4
        q, k, v = (t[0, :heads].cpu().float() for t in (self.q, self.k, self.v))
        scale = 1.0 / math.sqrt(self.dim)

        def run():
            return torch.softmax((q @ k.transpose(-1, -2)) * scale, dim=-1) @ v

        def compare(ref):
            self.o.fill_(float("nan"))
            self.step()
            return error_metrics(self.o[0, :heads], ref, f"batch 0, heads 0..{heads - 1} of O")

        return (run, 4.0 * heads * self.seq * self.seq * self.dim,
                f"1 batch x {heads} heads of {self.batch}x{self.heads} (fp32 torch softmax(QK^T)V), scaled by FLOPs", compare)


class LstmWorkload(Workload):
    name = "lstm"
    metric = "LSTM chain b256 i1024 h1024 x64 steps TFLOP/s"
    steps, batch, inp, hidden = 64, 256, 1024, 1024
    graph_steps = 1

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

    def e2e_tensors(self):
        return [self.w, self.u, self.x, self.h0, self.c0], [self.h_all, self.c_t]

    def cpu_reference(self):
        from oracle import oracle   # the CPU leg: the reference computation, also the checker of the launch below
        w, u, x, h0, c0 = (t.cpu() for t in (self.w, self.u, self.x, self.h0, self.c0))

        def run():
            return oracle.lstm_chain(w, u, None, x, h0, c0)

        def compare(ref):
            self.h_all.fill_(float("nan"))
            self.step()
            eh = error_metrics(self.h_all, ref[0], "h_t of all 64 steps")
            ec = error_metrics(self.c_t, ref[1], "c_T")
            return {"max_abs_err": max(eh["max_abs_err"], ec["max_abs_err"]), "rel_fro_err": max(eh["rel_fro_err"], ec["rel_fro_err"]),
                    "checked": "every h_t [64, 256, 1024] and c_T of the chain", "against": eh["against"]}

        return run, self.units_per_step(), "full 64-step chain (fp32 torch)", compare


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
        return {"table": "[2^26, 8] fp16", "updates": "2^24 unique rows", "indices": "int32",
                "l2": f"{self.rotate} rotating index/update sets (320 MB each) larger than L2", "flush_l2": False}

    def e2e_tensors(self):
        # the table is the state successive scatters update and stays on the device; a step brings its index and
        # update rows up and takes the updated table back
        return [self.idx[0], self.upd[0]], [self.table]

    def e2e_step(self):
        from tiledcuda_b200 import ops
        for dev, host in self._e2e_in:
            dev.copy_(host, non_blocking=True)
        ops.scatter_nd(self.table, self.idx[0], self.upd[0])
        for dev, host in self._e2e_out:
            host.copy_(dev, non_blocking=True)

    def cpu_reference(self):
        from tiledcuda_b200 import ops
        start = self.table.clone()          # whatever state the timed steps left: both sides start from it
        table = start.cpu()
        idx = self.idx[0].cpu().view(-1).long()
        upd = self.upd[0].cpu()

        def run():
            table[idx] = upd
            return table

        def compare(ref):
            ops.scatter_nd(start, self.idx[0], self.upd[0])
            same = torch.equal(start.cpu().view(torch.int16), ref.view(torch.int16))
            return {"bit_exact": bool(same), "checked": "the whole table after one scatter (2^26 x 8 fp16)",
                    "against": "torch index assignment on the CPU from the same starting table"}

        return run, self.units_per_step(), "full problem (torch index assignment)", compare


def make_workload(name: str) -> Workload:
    if name.startswith("gemm"):
        return GemmWorkload(int(name[4:]))
    return {"b2b": B2bWorkload, "fa": AttentionWorkload, "lstm": LstmWorkload, "scatter": ScatterWorkload}[name]()


def config_of(w: Workload, world: int) -> dict:
    """The `config` object; both arms print the same keys for the same workload and N."""
    return {"workload": w.name, **w.describe(), "parallelism": f"dp{world} (row slabs, no data-path collective)"}


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


def sustained_leg(w: Workload, ms_estimate: float, local_rank: int, peaks: dict, barrier, seconds: float = SUSTAINED_SECONDS) -> dict:
    """The step looped back to back for at least `seconds` of device time, with SM clock, power and throttle
    reasons sampled across the whole loop: long enough for the power governor to settle and for NVML's readings to
    describe the timed region. The fraction is taken against the sustained peak (a seconds-long cuBLAS loop), the
    like-for-like denominator for this leg and for no other."""
    steps = max(20, int(math.ceil(seconds * 1e3 / max(ms_estimate, 1e-3) * 1.1)))
    torch.cuda.synchronize()
    time.sleep(0.5)
    sampler = ClockSampler(local_rank)
    ms = time_steps(w.step, steps, 3, barrier, on_timed_start=sampler.start)
    clocks = sampler.stop()
    scale = 1e12 if w.unit == "TFLOP/s" else 1e9
    value = w.units_per_step() / (ms * 1e-3) / scale
    out = {"seconds": round(ms * steps / 1e3, 3), "steps": steps, "ms_per_step": round(ms, 4), "value": round(value, 2), "unit": w.unit,
           "sm_mhz_median": clocks.get("sm_mhz"), "sm_min_mhz": clocks.get("sm_min_mhz"), "power_w_max": clocks.get("power_w_max"),
           "reasons": clocks.get("reasons"), "clock_samples": clocks.get("samples"),
           "cycles_per_step": round(ms * 1e-3 * clocks["sm_mhz"] * 1e6) if clocks.get("sm_mhz") else None}
    if w.bound == "tensor":
        out["peak_sustained"] = peaks["tflops_sustained"]
        out["frac_of_sustained"] = round(value / peaks["tflops_sustained"], 4)
        out["frac_of_nominal"] = round(value / NOMINAL_TFLOPS, 4)
    return out


def roofline(w: Workload, ms: float, peaks: dict, burst_ms: float | None = None) -> dict:
    if w.bound == "tensor":
        achieved = w.units_per_step() / (ms * 1e-3) / 1e12
        peak, unit, nominal = peaks["tflops"], "TFLOP/s", NOMINAL_TFLOPS
    else:
        nbytes = w.bytes_per_step() if hasattr(w, "bytes_per_step") else w.units_per_step()
        achieved = nbytes / (ms * 1e-3) / 1e9
        peak, unit, nominal = peaks["hbm_gbs"], "GB/s", NOMINAL_HBM_GBS
    out = {"bound": w.bound, "achieved": round(achieved, 2), "peak": peak, "unit": unit, "frac": round(achieved / peak, 4),
           "peak_source": peaks["source"], "peak_kind": "burst (best of 10 isolated launches of the library kernel)" if w.bound == "tensor"
           else "stream copy", "frac_of_nominal": round(achieved / nominal, 4), "traffic": NCU_TRAFFIC_BYTES.get(w.name)}
    if burst_ms is not None and w.bound == "tensor":
        burst = w.units_per_step() / (burst_ms * 1e-3) / 1e12
        out.update({"achieved_burst": round(burst, 2), "frac_burst": round(burst / peak, 4),
                    "burst_how": "fastest of 10 single steps, each after a 50 ms idle pause"})
    return out


def cpu_and_parity(w: Workload, reps: int = 2) -> tuple[dict, dict]:
    """The CPU leg: the reference's computation of a bounded sample on all host cores, timed; its result is then
    the yardstick for one checked launch of the product op (outside every timed region)."""
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    run, units, sample, compare = w.cpu_reference()
    ref = run()
    best = float("inf")
    for _ in range(reps):
        t0 = time.perf_counter()
        ref = run()
        best = min(best, time.perf_counter() - t0)
    scale = 1e12 if w.unit == "TFLOP/s" else 1e9
    cpu = {"value": round(units / best / scale, 4), "unit": w.unit, "cores": threads, "kind": "port",
           "sample": sample, "seconds_per_sample": round(best, 4)}
    parity = compare(ref)
    torch.cuda.synchronize()
    return cpu, parity


def e2e_leg(w: Workload, steps: int, barrier, world: int, reduce_max) -> dict:
    w.e2e_setup()
    ms = reduce_max(time_steps(w.e2e_step, steps, 3, barrier))
    h2d, d2h = w.e2e_bytes()
    scale = 1e12 if w.unit == "TFLOP/s" else 1e9
    return {"value": round(w.units_per_step() * world / (ms * 1e-3) / scale, 3), "unit": w.unit, "h2d_bytes_per_step": h2d,
            "d2h_bytes_per_step": d2h, "ms_per_step": round(ms, 3), "steps": steps, "how": w.e2e_how()}


# ----------------------------------------------------------------------------------------------------
# the reference arm: the reference's CPU path on the host cores
# ----------------------------------------------------------------------------------------------------
def run_reference_arm(args, w: Workload, rank: int) -> int:
    """The reference's CPU path (its tests' torch fp32 computation) on the host cores; rank 0 only."""
    if rank != 0:
        return 0
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
    line = {
        "impl": "reference", "metric": w.metric, "value": value, "unit": w.unit, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(dt * 1e3, 3), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32 (torch CPU reference of the fp16 op)", "data": "synthetic",
        "config": config_of(w, args.gpus),
        "cpu_baseline": {"value": value, "unit": w.unit, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": w.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "reference_cuda_kernels": reference_cuda_kernels(),
    }
    print(json.dumps(line), flush=True)
    return 0


def reference_cuda_kernels() -> dict:
    """The reference's own CUDA kernels (sm_80-style cp.async / ldmatrix / mma.sync code compiled unmodified for
    sm_100a into oracle/_ref/ by oracle/ref_build/Makefile), run once each when they were built and a GPU is there.
    Kernels of the reference that cannot stand beside ours say why."""
    out: dict = {
        "fused_two_gemms": {"unavailable": "the reference's example binary ended with 'CUDA Runtime Error ... misaligned address' "
                                           "(fused_gemm.cu:117) on B200 after failing its own check at its second configuration; "
                                           "not run again on this pool"},
        "flash_attention": {"unavailable": "the reference's library kernel, run once on B200 through its own run_flash_attention at the "
                                           "largest shape its launcher supports (m 64, n 256, k = p = 128), ended with 'misaligned address'; "
                                           "not run again on this pool"},
        "scatter_nd": {"unavailable": "launcher defect in the reference: its launch passes the index buffer where the kernel expects "
                                      "the update values (src/kernels/scatter_nd.cu:107), so its result is not the op's"},
        "lstm_cell": {"unavailable": "the reference snapshot names the op (Makefile:3) but has no code for it"},
    }
    ref_dir = ROOT / "oracle" / "_ref"
    if not torch.cuda.is_available():
        out["gemm"] = {"unavailable": "no GPU in this process"}
        return out

    def run_binary(name):
        exe = ref_dir / name
        if not exe.exists():
            return None, f"{name} was not built (oracle/ref_build/Makefile, target ref_cuda)"
        try:
            res = subprocess.run([str(exe)], capture_output=True, text=True, timeout=180, cwd=str(ref_dir))
        except (OSError, subprocess.TimeoutExpired) as e:
            return None, type(e).__name__
        return res, None

    res, why = run_binary("ref_gemm_4096")
    if res is None:
        out["gemm_4096"] = {"unavailable": why}
    else:
        lines = [l for l in res.stdout.strip().splitlines() if l.strip()]
        try:
            cublas_ms, ref_ms, _ = (float(x) for x in lines[-1].split())
            flops = 2.0 * 4096 ** 3
            out["gemm_4096"] = {"workload": "fp16 GEMM 4096^3 (reference example 02_gemm_all_mem as it is, CTA tile 64x256x32)",
                                "self_check": "Test passed." in res.stdout, "ms": ref_ms, "tflops": round(flops / ref_ms / 1e9, 1),
                                "cublas_hgemm_ms": cublas_ms, "cublas_hgemm_tflops": round(flops / cublas_ms / 1e9, 1)}
        except (ValueError, IndexError):
            out["gemm_4096"] = {"unavailable": f"exit {res.returncode}: {(res.stdout + res.stderr)[-200:]}"}
    res, why = run_binary("ref_gemm_8192")
    if res is None:
        out["gemm_8192"] = {"unavailable": why}
    else:
        fields = dict(f.split("=", 1) for f in res.stdout.split() if "=" in f)
        try:
            out["gemm_8192"] = {"workload": "fp16 GEMM 8192^3: the reference's `gemm` kernel and KeGemmTraits instantiated at the headline "
                                            "size by a wrapper translation unit (same CTA tile 64x256x32), uniform[-1,1) inputs",
                                "ms": float(fields["ms"]), "tflops": float(fields["tflops"]), "self_check": fields.get("check") == "ok"}
        except (KeyError, ValueError):
            out["gemm_8192"] = {"unavailable": f"exit {res.returncode}: {(res.stdout + res.stderr)[-200:]}"}
    return out


def _cpu_only_sample(w: Workload):
    """CPU sample with inputs generated on the host (no GPU involved)."""
    if isinstance(w, GemmWorkload):
        n = w.n
        rows = cpu_rows_for(n)
        g = torch.Generator().manual_seed(SEED)
        b32 = (torch.rand(n, n, generator=g) * 2 - 1).half().float()
        a32 = (torch.rand(rows, n, generator=g) * 2 - 1).half().float()
        return (lambda: a32 @ b32.t()), 2.0 * rows * n * n, f"{rows} of {n} rows of A against the full B (fp32 torch matmul), scaled by FLOPs"
    w.setup(torch.device("cpu"), 0)
    if isinstance(w, B2bWorkload):
        a, b, d = w.a.float(), w.b.float(), w.d.float()
        return (lambda: ((a @ b.t()).half().float()) @ d.t()), w.units_per_step(), "full problem (fp32 torch, intermediate rounded to fp16)"
    if isinstance(w, AttentionWorkload):
        heads = 4
        q, k, v = (t[0, :heads].float() for t in (w.q, w.k, w.v))
        scale = 1.0 / math.sqrt(w.dim)
        return ((lambda: torch.softmax((q @ k.transpose(-1, -2)) * scale, dim=-1) @ v), 4.0 * heads * w.seq * w.seq * w.dim,
                f"1 batch x {heads} heads of {w.batch}x{w.heads} (fp32 torch softmax(QK^T)V), scaled by FLOPs")
    if isinstance(w, LstmWorkload):
        from oracle import oracle
        return (lambda: oracle.lstm_chain(w.w, w.u, None, w.x, w.h0, w.c0)), w.units_per_step(), "full 64-step chain (fp32 torch)"
    table, idx, upd = w.table, w.idx[0].view(-1).long(), w.upd[0]

    def run():
        table[idx] = upd
        return table

    return run, w.units_per_step(), "full problem (torch index assignment)"


# ----------------------------------------------------------------------------------------------------
# N > 1: the partitions of the path, through tiledcuda_b200/shard.py
# ----------------------------------------------------------------------------------------------------
def strong_gemm_leg(device, rank: int, world: int, barrier, reduce_max, steps: int) -> dict:
    """GEMM 16384^3 with the rows of A and C split across the ranks, B replicated, C assembled on every rank
    (all-gather over NVLink). Timed three ways: the slab products alone, the all-gather alone, and the overlapped
    form in which finished row blocks are exchanged from a side stream while later blocks compute. Efficiencies are
    against this run's own single-GPU time for the whole product, taken on rank 0 while the others wait."""
    import torch.distributed as dist
    from tiledcuda_b200 import ops, shard

    n = 16384
    g = torch.Generator(device=device).manual_seed(SEED)   # the same seed everywhere: replicated operands
    a = (torch.rand(n, n, generator=g, device=device) * 2 - 1).half()
    b = (torch.rand(n, n, generator=g, device=device) * 2 - 1).half()
    c = torch.empty(n, n, device=device)
    start, stop = shard.aligned_shard_range(n, world, rank, 128)

    single_ms = None
    if rank == 0:
        single_ms = time_steps(lambda: ops.gemm(a, b, c), max(3, steps // 2), 3, lambda: torch.cuda.synchronize())
    barrier()
    single_ms = broadcast_float(single_ms, device)

    compute_ms = reduce_max(time_steps(lambda: shard.sharded_gemm(a, b, c, gather=False), steps, 3, barrier))
    gather_ms = reduce_max(time_steps(lambda: shard.all_gather_slabs(c, world, rank), steps, 3, barrier))
    serial_ms = reduce_max(time_steps(lambda: shard.sharded_gemm(a, b, c, gather=True), steps, 3, barrier))
    best = None
    tried = []
    # Fewer, larger pushes keep the ranks' copy schedules in step for longer (on eight GPUs a rank's seven 128 MiB pushes
    # run at 680 GB/s, the same bytes in four or eight pieces per peer at 450 / 430 GB/s); more pieces start pushing earlier.
    for transport, blocks, max_sms, copy_streams in (("copy_engine", 4, 0, 1), ("copy_engine", 2, 0, 1), ("copy_engine", 8, 0, 1),
                                                    ("copy_engine", 4, 0, 2), ("nccl", 4, 132, 0)):
        if (stop - start) % (blocks * 128) != 0:
            continue
        try:
            op = shard.OverlappedGemm(blocks=blocks, max_sms=max_sms, transport=transport, copy_streams=copy_streams)
            ms = reduce_max(time_steps(lambda: op(a, b, c), steps, 3, barrier))
        except RuntimeError as e:   # CUDA IPC refused (a sandbox may not allow it): the NCCL transport remains
            tried.append({"transport": transport, "blocks": blocks, "unavailable": str(e)[:160]})
            continue
        if op.assembly is not None and op.assembly.windows is not None:
            torch.cuda.synchronize()
            op.assembly.windows.close()     # no rank keeps a window on C beyond this leg (C is freed below)
            barrier()
        tried.append({"transport": transport, "blocks": blocks, "gemm_sms": max_sms or "all",
                      **({"copy_streams": min(copy_streams, world - 1)} if transport == "copy_engine" else {}), "ms": round(ms, 4)})
        if best is None or ms < best[0]:
            best = (ms, blocks, max_sms, transport)
    # the assembled C of the last (overlapped) run against the product computed by one GPU: exact equality,
    # both come from the same kernels on the same operands
    torch.cuda.synchronize()
    check_rows = torch.arange(0, n, 997, device=device)
    got = c[check_rows].clone()
    ops.gemm(a[check_rows], b, c[: check_rows.numel()])
    assembled_ok = bool(torch.equal(got, c[: check_rows.numel()]))
    out = {"workload": "gemm16384 (M = N = K = 16384, rows of A and C split across ranks, C all-gathered to every rank)",
           "rows_per_gpu": stop - start, "single_gpu_ms": round(single_ms, 4), "compute_ms": round(compute_ms, 4),
           "gather_ms": round(gather_ms, 4), "compute_then_gather_ms": round(serial_ms, 4),
           "gather_bytes_received_per_gpu": (world - 1) * (stop - start) * n * 4,
           "gather_bus_gbs": round((world - 1) * (stop - start) * n * 4 / (gather_ms * 1e-3) / 1e9, 1),
           "efficiency_compute_only": round(single_ms / (world * compute_ms), 4),
           "assembled_rows_equal_single_gpu_product": assembled_ok,
           "collective": "NCCL all_gather_into_tensor (alone); overlapped: finished row blocks pushed into the peers' C by the copy "
                         "engines through CUDA IPC windows, or NCCL grouped send+recv beside a GEMM on fewer SMs"}
    if best is not None:
        out.update({"overlapped_ms": round(best[0], 4), "overlap_blocks": best[1], "overlap_gemm_sms": best[2] or "all",
                    "overlap_transport": best[3], "overlap_tried": tried,
                    "efficiency_end_to_end": round(single_ms / (world * best[0]), 4),
                    "bound_by": "NVLink ingress of the fp32 C all-gather" if gather_ms > compute_ms else "compute"})
    else:
        out["efficiency_end_to_end"] = round(single_ms / (world * serial_ms), 4)
    del a, b, c
    torch.cuda.empty_cache()
    return out


def broadcast_float(x, device) -> float:
    import torch.distributed as dist
    t = torch.tensor([x if x is not None else 0.0], device=device, dtype=torch.float64)
    dist.broadcast(t, src=0)
    return t.item()


def sharded_others(device, rank: int, world: int, barrier, reduce_max) -> dict:
    """Attention over batch x heads, the LSTM chain over batch and owner-computes scatter_nd, each split across the
    ranks by tiledcuda_b200/shard.py with no collective inside the timed region, and the same whole problem timed
    on rank 0 alone in the same run as the yardstick."""
    from tiledcuda_b200 import ops, shard
    out = {}
    alone = lambda: torch.cuda.synchronize()

    # ---- attention: 512 (batch, head) pairs, contiguous ranges per rank
    fa = AttentionWorkload()
    fa.setup(device, 0)                     # replicated operands (same seed on every rank)
    single = time_steps(fa.step, 5, 3, alone) if rank == 0 else None
    barrier()
    single = broadcast_float(single, device)
    ms = reduce_max(time_steps(lambda: shard.sharded_flash_attn(fa.q, fa.k, fa.v, fa.o, gather=False), 10, 3, barrier))
    pairs = fa.batch * fa.heads
    lo, hi = shard.shard_range(pairs, world, rank)
    gather_ms = reduce_max(time_steps(lambda: shard.all_gather_slabs(fa.o.view(pairs, fa.seq, fa.dim), world, rank), 5, 2, barrier))
    serial_ms = reduce_max(time_steps(lambda: shard.sharded_flash_attn(fa.q, fa.k, fa.v, fa.o, gather=True), 10, 3, barrier))
    out["fa"] = {"units": f"{pairs} (batch, head) pairs, {hi - lo} on this rank", "ms_sharded": round(ms, 4), "single_gpu_ms": round(single, 4),
                 "tflops_per_gpu": round(fa.units_per_step() / world / (ms * 1e-3) / 1e12, 1),
                 "efficiency": round(single / (world * ms), 4), "gather_of_O_ms": round(gather_ms, 4),
                 "ms_then_gather": round(serial_ms, 4),
                 "bound_by": "compute; the fp16 O all-gather (timed apart) is NVLink-ingress bound"}
    try:
        # every peer copy costs a fixed time on top of its bytes: fewer blocks win when there are many peers
        tried = {}
        for blocks in (4, 2):
            asm = shard.OverlappedAssembly(blocks=blocks)
            tried[blocks] = reduce_max(time_steps(lambda: shard.overlapped_flash_attn(asm, fa.q, fa.k, fa.v, fa.o), 10, 3, barrier))
            torch.cuda.synchronize()
            asm.windows.close()
            barrier()
        best_blocks = min(tried, key=tried.get)
        ov_ms = tried[best_blocks]
        out["fa"].update({"ms_with_O_assembled_overlapped": round(ov_ms, 4), "overlap_blocks": best_blocks,
                          "overlap_tried": {str(k): round(v, 4) for k, v in tried.items()},
                          "efficiency_with_O_assembled": round(single / (world * ov_ms), 4),
                          "overlap": "finished (batch, head) groups pushed into the peers' O by the copy engines (peer windows) "
                                     "while later groups are computed"})
    except RuntimeError as e:
        out["fa"]["overlap_unavailable"] = str(e)[:160]
    del fa
    torch.cuda.empty_cache()

    # ---- LSTM chain: batch rows split, weights replicated, no per-step communication
    lw = LstmWorkload()
    lw.setup(device, 0)
    single = time_steps(lw.step, 10, 3, alone, graph=1) if rank == 0 else None
    barrier()
    single = broadcast_float(single, device)
    lo, hi = shard.shard_range(lw.batch, world, rank)
    xs = lw.x[:, lo:hi].contiguous()
    hs = torch.empty(lw.steps, hi - lo, lw.hidden, dtype=torch.float16, device=device)
    cs = torch.empty(hi - lo, lw.hidden, device=device)
    ws = torch.empty(ops.lstm_chain_workspace_bytes(lw.steps, hi - lo, lw.hidden) // 4, device=device)
    chain = lambda: ops.lstm_chain(lw.w, lw.u, None, xs, lw.h0[lo:hi], lw.c0[lo:hi], hs, cs, workspace=ws)
    ms = reduce_max(time_steps(chain, 10, 3, barrier, graph=1))
    out["lstm"] = {"units": f"{lw.batch} batch rows, {hi - lo} on this rank", "ms_sharded": round(ms, 4), "single_gpu_ms": round(single, 4),
                   "tflops_per_gpu": round(lw.units_per_step() / world / (ms * 1e-3) / 1e12, 1),
                   "efficiency": round(single / (world * ms), 4),
                   "bound_by": "per-step latency: a step's time hardly depends on the batch rows a GPU holds"}
    del lw, xs, hs, cs, ws
    torch.cuda.empty_cache()

    # ---- scatter_nd: each rank owns a row range of the table and applies the updates that fall into it
    sw = ScatterWorkload()
    g = torch.Generator(device=device).manual_seed(SEED)
    idx = torch.randperm(sw.rows, generator=g, device=device)[: sw.n].to(torch.int32).view(-1, 1).contiguous()
    upd = torch.randn(sw.n, sw.width, generator=g, device=device, dtype=torch.float16)
    single = None
    if rank == 0:
        table = torch.zeros(sw.rows, sw.width, dtype=torch.float16, device=device)
        single = time_steps(lambda: ops.scatter_nd(table, idx, upd), 10, 3, alone)
        del table
    barrier()
    single = broadcast_float(single, device)
    r0, r1 = shard.shard_range(sw.rows, world, rank)
    slab = torch.zeros(r1 - r0, sw.width, dtype=torch.float16, device=device)
    # the updates are bucketed by owner once, outside the timed region
    rows = idx.view(-1)
    mine = (rows >= r0) & (rows < r1)
    local_idx = (rows[mine] - r0).to(torch.int32).view(-1, 1).contiguous()
    local_upd = upd[mine].contiguous()
    ms = reduce_max(time_steps(lambda: ops.scatter_nd(slab, local_idx, local_upd), 20, 3, barrier))
    out["scatter"] = {"units": f"{sw.rows} table rows, [{r0}, {r1}) owned by this rank ({r1 - r0} rows, {(r1 - r0) * 16 >> 20} MiB), "
                               f"{int(local_idx.shape[0])} of {sw.n} updates", "ms_sharded": round(ms, 4), "single_gpu_ms": round(single, 4),
                      "gbs_per_gpu": round(sw.units_per_step() / world / (ms * 1e-3) / 1e9, 1),
                      "efficiency": round(single / (world * ms), 4),
                      "bucketing": "updates assigned to owners once, outside the timed region",
                      "bound_by": "HBM / L2: an owner's slab is a fraction of the table, so its random rows fall into fewer DRAM pages"}
    return out


def sharded_e2e_leg(w: GemmWorkload, device, rank: int, world: int, barrier, reduce_max, steps: int) -> dict:
    """Host operands at N > 1: a rank uploads its own A slab and 1/N of B; the B slices are all-gathered over
    NVLink; C slabs go back to each rank's host buffer (tiledcuda_b200.shard.HostGemmPipeline)."""
    from tiledcuda_b200 import shard
    n = w.n
    pipe = shard.HostGemmPipeline(n, n, n, device, blocks=4)
    lo, hi = pipe.b_slice()
    h_a = w.a.cpu().pin_memory()
    h_b = w.b[lo:hi].cpu().pin_memory()
    h_c = torch.empty(n, n, dtype=torch.float32).pin_memory()
    ms = reduce_max(time_steps(lambda: pipe(h_a, h_b, h_c), steps, 3, barrier))
    torch.cuda.synchronize()
    # the slab that came back equals the device-side product of the same operands
    check = torch.empty(256, n, device=device)
    from tiledcuda_b200 import ops
    ops.gemm(w.a[:256], w.b, check)
    ok = bool(torch.equal(check.cpu(), h_c[:256]))
    return {"value": round(w.units_per_step() * world / (ms * 1e-3) / 1e12, 3), "unit": w.unit,
            "h2d_bytes_per_step": n * n * 2 + (hi - lo) * n * 2, "d2h_bytes_per_step": n * n * 4, "ms_per_step": round(ms, 3), "steps": steps,
            "how": "per rank: A slab and 1/N of B uploaded from pinned host memory, B all-gathered over NVLink (NCCL), block products, "
                   "C slab downloaded; three streams", "nvlink_bytes_received_per_step": (world - 1) * (hi - lo) * n * 2,
            "result_equals_device_product": ok}


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
    ap.add_argument("--no-others", action="store_true", help="skip the other workloads (N = 1) / the sharded ones (N > 1)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline and parity leg")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end leg")
    ap.add_argument("--no-sustained", action="store_true", help="skip the >= 2 s sustained leg")
    ap.add_argument("--no-strong", action="store_true", help="N > 1: skip the strong-scaling GEMM 16384^3 leg")
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
    affinity = None
    if distributed:
        import torch.distributed as dist
        affinity = bind_to_gpu_numa_node(local_rank)
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)
        barrier = lambda: (dist.barrier(), torch.cuda.synchronize())

        def reduce_max(ms: float) -> float:
            t = torch.tensor([ms], device=device, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return t.item()
    else:
        barrier = lambda: torch.cuda.synchronize()
        reduce_max = lambda ms: ms

    peaks = measured_peaks()
    w.setup(device, rank)
    desc = w.describe()
    scale = 1e12 if w.unit == "TFLOP/s" else 1e9

    sampler = ClockSampler(local_rank)
    ms = time_steps(w.step, args.steps, args.warmup, barrier, flush=bool(desc.get("flush_l2")), device=device,
                    on_timed_start=sampler.start, graph=w.graph_steps)
    clocks = sampler.stop()
    clocks["note"] = ("samples of the timed region only; a region of a few tens of milliseconds is shorter than NVML's own "
                      "averaging, see `sustained` for clocks that describe their loop")
    burst_ms = best_of_steps(w.step, 10, barrier) if (w.bound == "tensor" and w.launches_per_step() == 1) else None
    status = _lib.device_status()
    ms_max = reduce_max(ms)
    value = w.units_per_step() * world / (ms_max * 1e-3) / scale

    line = {
        "metric": w.metric, "value": round(value, 2), "unit": w.unit, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms_max, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": w.dtype, "data": "synthetic",
        "config": config_of(w, world),
        "roofline": roofline(w, ms, peaks, burst_ms),
        "clocks": clocks,
        "gpu_launches": (-(-args.steps // w.graph_steps) * w.graph_steps if w.graph_steps else args.steps) * w.launches_per_step(),
        "device_status": status,
    }
    if affinity is not None:
        line["host_affinity"] = affinity

    if not args.no_sustained and w.graph_steps == 0:
        s = sustained_leg(w, ms, local_rank, peaks, barrier)
        if distributed:
            s["ms_per_step"] = round(reduce_max(s["ms_per_step"]), 4)
            s["value"] = round(w.units_per_step() * world / (s["ms_per_step"] * 1e-3) / scale, 2)
            s.pop("frac_of_sustained", None)
            s.pop("frac_of_nominal", None)
            s["note"] = "whole-job value over the slowest rank; clocks are rank 0's"
        line["sustained"] = s

    if not args.no_e2e:
        e_steps = max(3, min(args.steps, 10))
        if distributed and isinstance(w, GemmWorkload):
            line["e2e"] = sharded_e2e_leg(w, device, rank, world, barrier, reduce_max, e_steps)
        elif not distributed:
            line["e2e"] = e2e_leg(w, e_steps, barrier, world, reduce_max)

    if distributed:
        if isinstance(w, GemmWorkload):
            # the all-gather that assembles the weak-scaling C on every rank, timed on its own
            from tiledcuda_b200 import shard
            full = torch.empty(world * w.n, w.n, device=device)
            full[rank * w.n:(rank + 1) * w.n].copy_(w.c)
            g_ms = reduce_max(time_steps(lambda: shard.all_gather_slabs(full, world, rank), max(3, args.steps // 4), 2, barrier))
            line["assemble"] = {"collective": "nccl all_gather of C (fp32)", "ms": round(g_ms, 4),
                                "bytes_received_per_gpu": (world - 1) * w.n * w.n * 4,
                                "bus_gbs": round((world - 1) * w.n * w.n * 4 / (g_ms * 1e-3) / 1e9, 1)}
            del full
        del w
        torch.cuda.empty_cache()
        if not args.no_strong:
            line["strong"] = strong_gemm_leg(device, rank, world, barrier, reduce_max, max(5, min(args.steps, 10)))
        if not args.no_others:
            line["others"] = sharded_others(device, rank, world, barrier, reduce_max)
        line["device_status_end"] = int(reduce_max(float(_lib.device_status())))
    else:
        if not args.no_cpu:
            line["cpu_baseline"], line["parity"] = cpu_and_parity(w)
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
                osampler = ClockSampler(local_rank)
                oms = time_steps(ow.step, ow.others_steps, 3, barrier, flush=bool(od.get("flush_l2")), device=device,
                                 on_timed_start=osampler.start, graph=ow.graph_steps)
                oscale = 1e12 if ow.unit == "TFLOP/s" else 1e9
                entry = {"metric": ow.metric, "value": round(ow.units_per_step() / (oms * 1e-3) / oscale, 2), "unit": ow.unit,
                         "ms_per_step": round(oms, 4), "steps": ow.others_steps, "roofline": roofline(ow, oms, peaks),
                         "launches_per_step": ow.launches_per_step(), "clocks": osampler.stop(), "config": config_of(ow, 1)}
                if name == "fa" and not args.no_sustained:
                    entry["sustained"] = sustained_leg(ow, oms, local_rank, peaks, barrier)
                if not args.no_cpu:
                    entry["cpu_baseline"], entry["parity"] = cpu_and_parity(ow, reps=1 if name == "scatter" else 2)
                others[name] = entry
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
