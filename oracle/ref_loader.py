"""Import the UNMODIFIED reference package (0xEodum/KAN) when its tree is present.

TEST INFRASTRUCTURE ONLY.  Used by the CPU tests that pin the restatement in
``chebykan_oracle.py`` and by ``tests/golden/make_golden.py``.  Nothing that
runs on a GPU box calls it: the reference tree does not travel there.

The reference's ``kan/__init__.py:33`` imports its plotting helpers
unconditionally and those import matplotlib, which is not installed in this
image.  Two stub modules are enough for the import to succeed; no reference
file is modified or copied.
"""
from __future__ import annotations

import os
import sys
import types



def reference_root() -> str | None:
    """Directory that holds the reference's ``kan`` package, or None."""
    cands = []
    if os.environ.get("KAN_REF"):
        cands.append(os.environ["KAN_REF"])
    cands.append(os.path.join(os.sep, "root", "reference"))
    for c in cands:
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
