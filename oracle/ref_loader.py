"""Import the UNMODIFIED reference package (0xEodum/KAN) when its tree is present.

TEST INFRASTRUCTURE ONLY.  Used by the CPU tests that pin the restatement in
``chebykan_oracle.py`` and by ``tests/golden/make_golden.py``, and by ``bench.py --impl reference``, which
times the reference itself when a tree is found and the restatement otherwise.

The reference's ``kan/__init__.py:33`` imports its plotting helpers
unconditionally and those import matplotlib, which is not installed in this
image.  Two stub modules are enough for the import to succeed; no reference
file is modified or copied.
"""
from __future__ import annotations

import os
import sys
import types



# Where the reference tree is looked for, in this order: the directory named by $KAN_REF, a copy under
# baseline/_ref/ at the repository root (git-ignored; present only where somebody put one), and the
# read-only mount the build container provides.  A box without any of them runs on the restatement alone.
_REPO_ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DEFAULT_MOUNT = os.path.join(os.sep, "root", "reference")


def candidate_roots() -> list:
    cands = []
    if os.environ.get("KAN_REF"):
        cands.append(os.environ["KAN_REF"])
    cands.append(os.path.join(_REPO_ROOT, "baseline", "_ref"))
    cands.append(DEFAULT_MOUNT)
    return cands


def reference_root() -> str | None:
    """Directory that holds the reference's ``kan`` package, or None."""
    for c in candidate_roots():
        if os.path.isfile(os.path.join(c, "kan", "layers", "chebykan.py")):
            return c
    return None


def available() -> bool:
    return reference_root() is not None


def load():
    """Return the reference's ``kan`` package (raises ImportError if absent)."""
    root = reference_root()
    if root is None:
        raise ImportError("reference tree not present on this machine")
    if "matplotlib" not in sys.modules:
        try:
            import matplotlib  # noqa: F401
        except Exception:
            mpl = types.ModuleType("matplotlib")
            plt = types.ModuleType("matplotlib.pyplot")
            plt.Figure = type("Figure", (), {})
            mpl.pyplot = plt
            sys.modules["matplotlib"] = mpl
            sys.modules["matplotlib.pyplot"] = plt
    if root not in sys.path:
        sys.path.insert(0, root)
    import kan  # noqa: E402
    return kan


def reference_layer_cls():
    load()
    from kan.layers.chebykan import ChebyKANLayer
    return ChebyKANLayer
