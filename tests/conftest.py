import os
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def golden_codec():
    return np.load(os.path.join(GOLDEN, "codec.npz"))


@pytest.fixture(scope="session")
def golden_layer():
    return np.load(os.path.join(GOLDEN, "layer.npz"))


@pytest.fixture(scope="session")
def golden_decode_table():
    return np.load(os.path.join(GOLDEN, "decode_q4_exhaustive.npz"))["twice_residual"]


def bits(a):
    """float32 array -> uint32 view for bit-exact comparison (+0.0 and -0.0 unified)."""
    a = np.ascontiguousarray(a, dtype=np.float32) + np.float32(0.0)
    return a.view(np.uint32)
