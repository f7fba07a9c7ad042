"""Shared test set-up: the ``gpu`` marker, the repo root on ``sys.path`` and small helpers."""

import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
for entry in (ROOT, ROOT / "tests"):
    if str(entry) not in sys.path:
        sys.path.insert(0, str(entry))
GOLDEN = ROOT / "tests" / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def golden():
    def load(name):
        return np.load(GOLDEN / f"{name}.npz")
    return load


@pytest.fixture(scope="session")
def cuda():
    """The CUDA device, with the native library loaded.  GPU tests fail, not skip, without it."""
    import torch

    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    from keep_b200 import _lib

    _lib.load()
    return torch.device("cuda", 0)
