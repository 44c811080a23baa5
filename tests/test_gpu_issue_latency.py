"""Runs the MMA issue-latency microbenchmark (tests/cpp/mma_issue_latency.cu) and checks the facts the kernels'
stage sizes rest on: between short MMAs a barrier wait on a completed phase is paid in full, wide MMAs hide it."""
import re
import subprocess
from pathlib import Path

import pytest

BIN = Path(__file__).resolve().parent / "cpp" / "mma_issue_latency"


@pytest.mark.gpu
def test_barrier_waits_between_short_mmas_are_exposed_and_wide_mmas_hide_them():
    if not BIN.exists():
        from tiledcuda_b200 import build
        build.build_tile_api_tests()
    res = subprocess.run([str(BIN)], capture_output=True, text=True, timeout=120)
    assert res.returncode == 0, res.stdout + res.stderr
    cycles = {}
    for m in re.finditer(r"N=(\d+) mmas_per_group=(\d+) between=(\w+) cycles_per_group=(\d+) status=(\d+)", res.stdout):
        assert m.group(5) == "0"
        cycles[(int(m.group(1)), int(m.group(2)), m.group(3))] = int(m.group(4))
    assert len(cycles) == 15, res.stdout
    # pipe rate: about 48 / 64 / 128 cycles per MMA for N = 64 / 128 / 256
    assert 180 <= cycles[(64, 4, "nothing")] <= 260
    assert 230 <= cycles[(128, 4, "nothing")] <= 300
    assert 480 <= cycles[(256, 4, "nothing")] <= 560
    # a commit or a tcgen05 fence is cheap, a wait on a completed phase is not
    assert cycles[(64, 4, "commit")] <= cycles[(64, 4, "nothing")] + 100
    assert cycles[(64, 4, "fence")] <= cycles[(64, 4, "nothing")] + 40
    assert cycles[(64, 4, "try_wait")] >= cycles[(64, 4, "nothing")] + 100
    assert cycles[(128, 4, "ring")] >= cycles[(128, 4, "nothing")] + 100
    # the cost is per wait, so longer groups amortise it, and 128-cycle MMAs hide it
    assert cycles[(64, 16, "try_wait")] / 16 < cycles[(64, 4, "try_wait")] / 4 * 0.8
    assert cycles[(256, 4, "ring")] <= cycles[(256, 4, "nothing")] * 1.1
