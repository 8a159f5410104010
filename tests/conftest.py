import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


@pytest.fixture(scope="session")
def orc():
    """The CPU oracle (oracle/oracle.c through ctypes), built on demand."""
    from oracle import binding
    binding.build()
    return binding


@pytest.fixture(scope="session")
def pins():
    return np.load(os.path.join(ROOT, "tests", "golden", "reference_pins.npz"))


@pytest.fixture(scope="session")
def cuda():
    """torch + the product package on a B200; GPU tests fail (not skip) without
    the native library, so a silent fallback cannot pass."""
    import torch
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    import llmp_b200
    assert llmp_b200.available(), llmp_b200._native.last_error()
    return torch
