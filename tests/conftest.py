"""pytest configuration: the `gpu` marker and shared fixtures."""
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = ROOT / "tests" / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def golden_ops():
    return dict(np.load(GOLDEN / "triton_ops.npz"))


@pytest.fixture(scope="session")
def golden_block():
    return dict(np.load(GOLDEN / "block_config1.npz"))


@pytest.fixture(scope="session")
def cuda():
    """A CUDA device with the kernel library loaded; GPU tests fail (not skip) if either is missing."""
    import torch

    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    from dejavu_b200 import _lib

    _lib.load()
    return torch.device("cuda:0")
