"""Generate golden vectors from the UNMODIFIED reference (0xEodum/KAN).

Run in a container where the reference tree is importable:
    python tests/golden/make_golden.py
It imports the reference's ``kan.layers.chebykan.ChebyKANLayer`` through
``oracle/ref_loader.py`` (matplotlib stub only; no reference file is modified
or copied), evaluates forward and autograd backward on seeded inputs on the
CPU, and writes ``tests/golden/chebykan_golden.npz``.  The fixtures let
machines without the reference tree (the GPU boxes) check both the oracle
restatement and the CUDA kernels against the reference's own outputs.
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import ref_loader  # noqa: E402

# name: (B-shape, in, out, degree, distribution, use_recurrence)
CASES = {
    "tiny_d4": ((37,), 5, 3, 4, "normal", False),
    "mid_d8": ((64,), 16, 8, 8, "normal", False),
    "cfg1_shape": ((100,), 1, 1, 8, "linspace", False),
    "deg32_uniform": ((33,), 7, 5, 32, "uniform3", False),
    "deg0": ((19,), 3, 2, 0, "normal", False),
    "deg1": ((19,), 3, 2, 1, "normal", False),
    "three_dim_input": ((2, 5), 4, 3, 3, "normal", False),
    "recurrence_path": ((41,), 6, 4, 8, "normal", True),
    "sparse_784": ((16,), 784, 10, 4, "sparse", False),
    "wide_out": ((9,), 12, 130, 4, "normal", False),
    "kat_points": ((3,), 1, 1, 4, "kat", False),
}


def make_x(shape, n_in, dist, g):
    full = tuple(shape) + (n_in,)
    if dist == "normal":
        return torch.randn(full, generator=g)
    if dist == "uniform3":
        return torch.rand(full, generator=g) * 6 - 3
    if dist == "linspace":
        return torch.linspace(-1, 1, shape[0], dtype=torch.float64).float().view(full)
    if dist == "sparse":
        x = torch.rand(full, generator=g)
        return torch.where(torch.rand(full, generator=g) < 0.8, torch.zeros(()), x)
    if dist == "kat":
        return torch.tensor([0.0, 8.0, -8.0]).view(full)
    raise KeyError(dist)


def main():
    Ref = ref_loader.reference_layer_cls()
    out = {}
    for idx, (name, (shape, n_in, n_out, deg, dist, rec)) in enumerate(sorted(CASES.items())):
        torch.manual_seed(4242 + idx)
        layer = Ref(n_in, n_out, deg, use_recurrence=rec)
        if name == "kat_points":
            with torch.no_grad():
                layer.cheby_coeffs.copy_(torch.ones_like(layer.cheby_coeffs))
        g = torch.Generator().manual_seed(777 + idx)
        # The reference's use_recurrence=True path writes slices in place, and its
        # autograd backward raises when x requires grad; only dC exists there.
        x = make_x(shape, n_in, dist, g).requires_grad_(not rec)
        y = layer(x)
        dy = torch.randn(y.shape, generator=g)
        y.backward(dy)
        out[f"{name}/x"] = x.detach().numpy()
        out[f"{name}/coeffs"] = layer.cheby_coeffs.detach().numpy()
        out[f"{name}/dy"] = dy.numpy()
        out[f"{name}/y"] = y.detach().numpy()
        out[f"{name}/dC"] = layer.cheby_coeffs.grad.numpy()
        if not rec:
            out[f"{name}/dx"] = x.grad.numpy()
        out[f"{name}/meta"] = np.array([n_in, n_out, deg, int(rec)], dtype=np.int64)
    # the README training loop (configuration 1): loss at fixed steps, seed 0
    torch.manual_seed(0)
    layer = Ref(1, 1, 8)
    xs = torch.linspace(-1, 1, 100, dtype=torch.float64).float().view(100, 1)
    tgt = torch.sin(2 * np.pi * xs)
    opt = torch.optim.Adam(layer.parameters(), lr=0.01)
    losses = []
    init = layer.cheby_coeffs.detach().clone().numpy()
    for step in range(1000):
        opt.zero_grad()
        loss = torch.nn.functional.mse_loss(layer(xs), tgt)
        loss.backward()
        opt.step()
        if step in (0, 99, 499, 999):
            losses.append(float(loss.detach()))
    out["cfg1_train/init_coeffs"] = init
    out["cfg1_train/final_coeffs"] = layer.cheby_coeffs.detach().numpy()
    out["cfg1_train/losses"] = np.array(losses, dtype=np.float64)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "chebykan_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes;", len(CASES), "cases; cfg1 losses", losses)


if __name__ == "__main__":
    main()
