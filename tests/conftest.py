import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = Path(__file__).resolve().parent / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100); run with -m gpu on a B200")


@pytest.fixture(scope="session")
def golden_dir():
    return GOLDEN


@pytest.fixture(scope="session")
def cuda_ops():
    """The product ops on cuda:0. Fails (never skips to a fallback) if the native library is missing."""
    import torch

    assert torch.cuda.is_available(), "gpu tests need a CUDA device"
    from tiledcuda_b200 import _lib, ops

    _lib.load()
    torch.cuda.set_device(0)
    return ops


@pytest.fixture()
def clean_status():
    """Checks that no kernel recorded a timeout or an out-of-range index during the test."""
    from tiledcuda_b200 import _lib

    yield
    assert _lib.device_status() == 0
