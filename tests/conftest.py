import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def golden():
    return np.load(ROOT / "tests" / "golden" / "aten_cpu.npz")


@pytest.fixture(scope="session")
def golden_rowops():
    return np.load(ROOT / "tests" / "golden" / "aten_cpu_rowops.npz")


@pytest.fixture(scope="session")
def cuda():
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from torchvulkan_b200 import capi

    capi.lib()  # fails loudly if the extension is not built
    return torch.device("cuda:0")


def rel_fro(a, b):
    """Relative Frobenius error ||a - b|| / ||b|| in float64."""
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    d = np.linalg.norm((a - b).ravel())
    n = np.linalg.norm(b.ravel())
    return d / n if n > 0 else d
