import importlib
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def golden():
    import numpy as np
    return np.load(os.path.join(ROOT, "tests", "golden", "golden.npz"))


@pytest.fixture(scope="session")
def q4t():
    """The product package (directory name carries a hyphen, hence importlib)."""
    return importlib.import_module("qwen4-thor_b200")


@pytest.fixture(scope="session")
def gpu_lib(q4t):
    """The loaded CUDA library; GPU tests fail loudly if it is missing."""
    import torch
    assert torch.cuda.is_available(), "GPU test selected but no CUDA device"
    return q4t.load()
