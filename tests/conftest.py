import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "craftax.cu_b200"))
sys.path.insert(0, os.path.join(ROOT, "oracle"))
GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def oracle():
    import oracle as O
    O.lib()
    return O


@pytest.fixture(scope="session")
def golden_env():
    d = np.load(os.path.join(GOLDEN, "env_rollout_seed0.npz"))
    return {k: d[k] for k in d.files}


@pytest.fixture(scope="session")
def golden_oracle():
    d = np.load(os.path.join(GOLDEN, "oracle_forward_seed0.npz"))
    return {k: d[k] for k in d.files}


@pytest.fixture(scope="session")
def cfx():
    """The ctypes binding; building the library is part of the product build, the tests
    only load it."""
    import cfx as m
    if not os.path.exists(m.LIB_PATH):
        sys.path.insert(0, os.path.join(ROOT, "craftax.cu_b200"))
        import build
        build.build()
    m.lib()
    return m


@pytest.fixture(scope="session")
def gpu(cfx):
    if cfx.device_count() < 1:
        pytest.fail("test marked gpu but no CUDA device is visible")
    return cfx.device_info(0)
