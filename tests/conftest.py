import os
import sys

import pytest

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100a) and the built CUDA library")


@pytest.fixture(scope="session")
def golden():
    """Outputs of the reference's own seblas kernels (recorded by tests/golden/make_golden.py)."""
    import numpy as np
    path = os.path.join(ROOT, "tests", "golden", "ref_seblas_golden.npz")
    if not os.path.exists(path):
        pytest.skip("golden vectors not recorded yet")
    return dict(np.load(path))


@pytest.fixture(scope="session")
def cuda_lib():
    """The C ABI library; GPU tests fail loudly (not skip) when it is missing."""
    from crusaderbackend_b200 import _lib
    return _lib.load()
