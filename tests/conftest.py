import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def golden(name):
    return np.load(os.path.join(GOLDEN, name), allow_pickle=False)


def bits(a):
    """fp32 array -> its bit patterns, so comparisons are bit-exact and NaN-safe."""
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


@pytest.fixture(scope="session")
def gold_softstep():
    return golden("softstep.npz")


@pytest.fixture(scope="session")
def gold_pack():
    return golden("pack.npz")


@pytest.fixture(scope="session")
def gold_codec():
    return golden("codec.npz")


@pytest.fixture(scope="session")
def gold_schedule():
    return golden("schedule.npz")


@pytest.fixture(scope="session")
def gold_mlp():
    return golden("mlp_step.npz")
