"""Helpers shared by the GPU parity tests."""
import torch
import torch.nn as nn

from oracle import chebykan_oracle as o

FP32_TOL = 1e-5    # rel-L2, fp32 FFMA mode, TF32 disabled
TC_TOL = 2e-3      # rel-L2, tf32 / bf16 tensor-core modes
GUARD = 1024       # floats of guard band on both sides of an output buffer
CANARY = 12345.0


class OracleLayer(nn.Module):
    """nn.Module wrapper over the oracle's forward, for model-level comparisons on the CPU."""

    def __init__(self, input_dim, output_dim, degree):
        super().__init__()
        self.input_dim = input_dim
        self.cheby_coeffs = nn.Parameter(o.init_coeffs(input_dim, output_dim, degree))

    def forward(self, x):
        return o.forward(x.view(-1, self.input_dim), self.cheby_coeffs)


def guarded(shape, device="cuda"):
    """(view, whole) — a NaN-poisoned output view inside a canary-filled buffer."""
    n = 1
    for s in shape:
        n *= s
    whole = torch.full((n + 2 * GUARD,), CANARY, dtype=torch.float32, device=device)
    view = whole[GUARD:GUARD + n].view(*shape)
    view.fill_(float("nan"))
    return view, whole


def assert_guards_intact(view, whole):
    n = view.numel()
    assert bool((whole[:GUARD] == CANARY).all()) and bool((whole[GUARD + n:] == CANARY).all()), \
        "kernel wrote outside its output buffer"
    assert not bool(torch.isnan(view).any()), "kernel left part of its output unwritten"


def make_case(B, n_in, n_out, deg, dist="normal", seed=0, sparse=False):
    g = torch.Generator().manual_seed(seed)
    if dist == "normal":
        x = torch.randn(B, n_in, generator=g)
    elif dist == "uniform3":
        x = torch.rand(B, n_in, generator=g) * 6 - 3
    elif dist == "sparse":
        x = torch.rand(B, n_in, generator=g)
        x = torch.where(torch.rand(B, n_in, generator=g) < 0.8, torch.zeros(()), x)
    else:
        raise KeyError(dist)
    coeffs = torch.randn(n_in, n_out, deg + 1, generator=g) / (n_in * (deg + 1))
    dy = torch.randn(B, n_out, generator=g)
    return x, coeffs, dy
