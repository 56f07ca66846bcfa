import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def load_golden(name):
    return np.load(os.path.join(GOLDEN, name + ".npz"))


def golden_cache(z, prefix):
    """Rebuild a 42-slot cache tuple of numpy arrays from a fixture."""
    out = [None] * 42
    for i in range(42):
        key = f"{prefix}_{i}"
        if key in z.files:
            out[i] = int(z[key]) if i == 41 else z[key]
    return tuple(out)


@pytest.fixture(scope="session")
def cuda_device():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")
