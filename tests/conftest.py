import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


@pytest.fixture(scope="session")
def golden():
    def load(name):
        return np.load(os.path.join(GOLDEN, name + ".npz"))
    return load


@pytest.fixture(scope="session")
def native_lib():
    """The built C-ABI library; compiled here when nvcc is present and it is stale."""
    import fast_transformers_b200  # noqa: F401
    from fast_transformers_b200 import build
    try:
        build.build()
    except Exception:
        if not os.path.exists(build.LIB):
            raise
    from fast_transformers_b200 import _native
    return _native.lib()
