import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.dirname(os.path.abspath(__file__))):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def golden():
    import numpy as np
    path = os.path.join(ROOT, "tests", "golden", "csg_golden.npz")
    return np.load(path)


@pytest.fixture(scope="session")
def built_lib():
    """The CUDA library, built if a source is newer (nvcc cross-compiles without a GPU)."""
    from chunkedgreedy_b200 import build
    return build.build()
