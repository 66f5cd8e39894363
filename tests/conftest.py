"""pytest configuration: registers the `gpu` marker and shared fixtures."""
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def oracle():
    from oracle_lib import load_oracle
    return load_oracle()


@pytest.fixture(scope="session")
def golden():
    import numpy as np
    path = os.path.join(ROOT, "tests", "golden", "kvpath_golden.npz")
    return dict(np.load(path))


@pytest.fixture(scope="session")
def layer_golden():
    """Vectors of tests/golden/gen_layer_golden.py (RMSNorm rows, sigmoid, the layer form of the step)."""
    import numpy as np
    path = os.path.join(ROOT, "tests", "golden", "layer_golden.npz")
    return dict(np.load(path))


@pytest.fixture(scope="session")
def bk():
    """The package (its directory name has a '-', hence importlib)."""
    import importlib
    return importlib.import_module("ternary-bonsai-inference_b200")


@pytest.fixture(scope="session")
def gpu_ctx(bk):
    return bk.Context(0)
