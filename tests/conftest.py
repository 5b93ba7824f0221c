import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def golden_codec():
    import numpy as np
    return dict(np.load(os.path.join(ROOT, "tests", "golden", "codec.npz")))


@pytest.fixture(scope="session")
def golden_gemm():
    import numpy as np
    return dict(np.load(os.path.join(ROOT, "tests", "golden", "gemm.npz")))


@pytest.fixture(scope="session")
def gemm_cases():
    import cases
    return cases.gemm_cases()
