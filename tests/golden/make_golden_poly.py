"""Generate golden vectors of the reference's Jacobi and Hermite layers from the UNMODIFIED reference.

Run in a container where the reference tree is importable:
    python tests/golden/make_golden_poly.py
It imports ``kan.layers.jacobikan.JacobiKANLayer`` and ``kan.layers.hermitekan.HermiteKANLayer`` through
``oracle/ref_loader.py`` (matplotlib stub only; no reference file is modified or copied), evaluates forward and
autograd backward on seeded inputs on the CPU and writes ``tests/golden/polykan_golden.npz``.  Machines without the
reference tree (the GPU boxes) check the oracle restatement and the CUDA kernels against these outputs.
"""
import json
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import ref_loader  # noqa: E402

# name: (rows, in, out, degree, x distribution, layer kind, constructor keywords)
CASES = {
    "legendre_d6": (37, 5, 3, 6, "normal", "jacobi", {}),
    "jacobi_a05_bm03_d9": (41, 7, 5, 9, "normal", "jacobi", {"alpha": 0.5, "beta": -0.3}),
    "jacobi_a2_b1_d16": (33, 6, 4, 16, "uniform3", "jacobi", {"alpha": 2.0, "beta": 1.0}),
    "jacobi_cheb1_d8": (29, 4, 4, 8, "normal", "jacobi", {"alpha": -0.5, "beta": -0.5}),
    "jacobi_d0": (19, 3, 2, 0, "normal", "jacobi", {}),
    "jacobi_d1": (19, 3, 2, 1, "normal", "jacobi", {"alpha": 1.0, "beta": 0.25}),
    "jacobi_wide_out": (9, 12, 130, 4, "normal", "jacobi", {"alpha": 0.0, "beta": 0.5}),
    "hermite_phys_d6": (37, 5, 3, 6, "normal", "hermite", {}),
    "hermite_prob_d9": (41, 7, 5, 9, "normal", "hermite", {"scaling": "probabilist"}),
    "hermite_phys_d12_uniform": (33, 6, 4, 12, "uniform3", "hermite", {}),
    "hermite_domain_affine": (31, 4, 3, 5, "uniform_dom", "hermite", {"domain": (-2.0, 5.0)}),
    "hermite_domain_no_normalize": (31, 4, 3, 5, "normal", "hermite", {"domain": (-2.0, 5.0), "normalize_domain": False}),
    "hermite_d0": (19, 3, 2, 0, "normal", "hermite", {}),
    "hermite_d1": (19, 3, 2, 1, "normal", "hermite", {"scaling": "probabilist"}),
}


def make_x(rows, n_in, dist, g):
    if dist == "normal":
        return torch.randn(rows, n_in, generator=g)
    if dist == "uniform3":
        return torch.rand(rows, n_in, generator=g) * 6 - 3
    if dist == "uniform_dom":
        return torch.rand(rows, n_in, generator=g) * 7 - 2
    raise KeyError(dist)


def main():
    ref_loader.load()
    from kan.layers.jacobikan import JacobiKANLayer
    from kan.layers.hermitekan import HermiteKANLayer
    out = {}
    for idx, (name, (rows, n_in, n_out, deg, dist, kind, kw)) in enumerate(sorted(CASES.items())):
        torch.manual_seed(9090 + idx)
        layer = (JacobiKANLayer if kind == "jacobi" else HermiteKANLayer)(n_in, n_out, deg, **kw)
        coeffs = layer.get_coefficients()
        g = torch.Generator().manual_seed(333 + idx)
        x = make_x(rows, n_in, dist, g).requires_grad_(True)
        y = layer(x)
        dy = torch.randn(y.shape, generator=g)
        y.backward(dy)
        # the oracle's description of the family (oracle/polykan_oracle.py: forward(family, x, coeffs))
        out[f"{name}/family"] = np.array(json.dumps(dict(kw, kind=kind)))
        out[f"{name}/x"] = x.detach().numpy()
        out[f"{name}/coeffs"] = coeffs.detach().numpy()
        out[f"{name}/dy"] = dy.numpy()
        out[f"{name}/y"] = y.detach().numpy()
        out[f"{name}/dC"] = coeffs.grad.numpy()
        # at degree 0 the output does not depend on x and autograd leaves x.grad unset
        out[f"{name}/dx"] = (x.grad if x.grad is not None else torch.zeros_like(x)).numpy()
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "polykan_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes;", len(CASES), "cases")


if __name__ == "__main__":
    main()
