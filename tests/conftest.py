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
def golden_poly():
    """Outputs of the unmodified reference's Jacobi and Hermite layers (tests/golden/make_golden_poly.py)."""
    return load_golden_poly()


def load_golden_poly():
    import json
    data = np.load(os.path.join(ROOT, "tests", "golden", "polykan_golden.npz"))
    cases = {}
    for key in data.files:
        name, field = key.split("/")
        cases.setdefault(name, {})[field] = data[key]
    for c in cases.values():
        fam = json.loads(str(c["family"]))
        if fam.get("domain") is not None:
            fam["domain"] = tuple(fam["domain"])
        c["family"] = fam
    return cases


@pytest.fixture(scope="session")
def built_lib():
    """Build the shared library in-tree if it is missing (nvcc cross-compiles without a GPU)."""
    from kan_b200 import _lib, build
    if not os.path.exists(_lib.LIB_PATH):
        build.build()
    return _lib.LIB_PATH
