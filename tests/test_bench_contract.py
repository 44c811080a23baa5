"""CPU tests of bench.py's contract: the reference arm prints one JSON line with the keys the driver reads, both arms
describe a workload with the same `config`, and the helper arithmetic (rotation sets, CPU sample sizes, roofline) is
what the documentation says. No GPU is touched."""
import importlib.util
import json
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def bench():
    spec = importlib.util.spec_from_file_location("bench_under_test", ROOT / "bench.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_reference_arm_prints_one_json_line_with_the_contract_keys():
    res = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--workload", "b2b", "--steps", "2", "--warmup", "1"],
                         capture_output=True, text=True, timeout=300, cwd=str(ROOT))
    assert res.returncode == 0, res.stderr[-500:]
    lines = [l for l in res.stdout.splitlines() if l.strip()]
    assert len(lines) == 1
    d = json.loads(lines[0])
    for key in ("impl", "metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "vs_baseline", "dtype", "data", "config", "cpu_baseline", "e2e", "gpu_launches", "reference_cuda_kernels"):
        assert key in d, key
    assert d["impl"] == "reference" and d["vs_baseline"] is None and d["value"] > 0
    assert d["e2e"] == {"value": d["value"], "unit": d["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["cores"] >= 1
    # the reference's kernels that cannot stand beside ours say why
    for name in ("fused_two_gemms", "flash_attention", "scatter_nd", "lstm_cell"):
        assert "unavailable" in d["reference_cuda_kernels"][name]


@pytest.mark.parametrize("name", ["gemm8192", "gemm1024", "b2b", "fa", "lstm", "scatter"])
def test_both_arms_describe_a_workload_with_the_same_config(bench, name):
    ours, theirs = bench.make_workload(name), bench.make_workload(name)
    for world in (1, 8):
        assert bench.config_of(ours, world) == bench.config_of(theirs, world)
        assert bench.config_of(ours, world)["workload"] == name and "parallelism" in bench.config_of(ours, world)


def test_small_workloads_rotate_through_more_than_l2(bench):
    assert bench.rotation_sets(8192 * 8192 * 8) == 1
    sets = bench.rotation_sets(1024 * 1024 * 8)
    assert sets * 1024 * 1024 * 8 > 126e6
    assert bench.GemmWorkload(1024).graph_steps == sets and bench.GemmWorkload(8192).graph_steps == 0
    assert bench.cpu_rows_for(8192) % 128 == 0 and bench.cpu_rows_for(1024) == 1024 and bench.cpu_rows_for(16384) >= 128


def test_roofline_uses_algorithmic_work_and_the_right_peak(bench):
    peaks = {"tflops": 1650.3, "tflops_sustained": 1386.1, "hbm_gbs": 6537.3, "source": "measured"}
    r = bench.roofline(bench.GemmWorkload(8192), 0.75, peaks, burst_ms=0.74)
    assert r["bound"] == "tensor" and r["unit"] == "TFLOP/s" and r["peak"] == 1650.3
    assert abs(r["achieved"] - 2 * 8192 ** 3 / 0.75e-3 / 1e12) < 0.01 and abs(r["frac"] - r["achieved"] / 1650.3) < 1e-3
    assert "frac_of_sustained" not in r          # that fraction belongs to the >= 2 s leg only
    s = bench.roofline(bench.ScatterWorkload(), 0.75, peaks)
    assert s["bound"] == "hbm" and s["unit"] == "GB/s" and abs(s["achieved"] - (1 << 24) * 36 / 0.75e-3 / 1e9) < 0.01
