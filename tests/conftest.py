import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 GPU (run with -m gpu)")


@pytest.fixture(scope="session")
def golden():
    """Outputs of the unmodified reference on seeded inputs (tests/golden/make_golden.py)."""
    path = os.path.join(ROOT, "tests", "golden", "chebykan_golden.npz")
    data = np.load(path)
    cases = {}
    for key in data.files:
        name, field = key.split("/")
        cases.setdefault(name, {})[field] = data[key]
    return cases


@pytest.fixture(scope="session")
def built_lib():
    """Build the shared library in-tree if it is missing (nvcc cross-compiles without a GPU)."""
    from kan_b200 import _lib, build
    if not os.path.exists(_lib.LIB_PATH):
        build.build()
    return _lib.LIB_PATH
