"""CPU restatement of the reference's Jacobi and Hermite KAN layers (0xEodum/KAN).

TEST INFRASTRUCTURE ONLY: imported by tests/, by tests/golden/make_golden_poly.py and by nothing in the
product path.  Same role as chebykan_oracle.py: the arithmetic of the reference, operation for operation,
in PyTorch on the CPU, so that results are bit-identical to the reference's own (tests/test_oracle_poly.py
pins that against the reference tree when it is present and against committed golden vectors otherwise).

    Jacobi   kan/basis/jacobi.py:84-96 (tanh), :136-188 (recurrence), :98-120 (einsum 'bid,iod->bo');
             kan/layers/jacobikan.py:20-68 (layer: parameter jacobi_coeffs[in, out, deg+1])
    Hermite  kan/basis/hermite.py:85-116 (3 tanh x, or the affine map of a finite domain onto [-3, 3]),
             :163-196 (physicist), :198-233 (probabilist), :118-141 (einsum);
             kan/layers/hermitekan.py:22-83 (layer: parameter hermite_coeffs[in, out, deg+1])
The reference has no hand-written backward: gradients are what autograd derives from these forwards.
"""
from __future__ import annotations

import math

import torch


def init_coeffs(input_dim: int, output_dim: int, degree: int, init_scale: float | None = None) -> torch.Tensor:
    """Same draw from the global CPU RNG as both layers' constructors (jacobikan.py:59-63, hermitekan.py:61-65)."""
    std = init_scale or 1.0 / (input_dim * (degree + 1))
    c = torch.empty(input_dim, output_dim, degree + 1)
    torch.nn.init.normal_(c, mean=0.0, std=std)
    return c


# ---------------------------------------------------------------------------------------------------------------
# Jacobi
# ---------------------------------------------------------------------------------------------------------------
def jacobi_basis(t: torch.Tensor, degree: int, alpha: float = 0.0, beta: float = 0.0) -> torch.Tensor:
    """P_0..P_degree^(alpha,beta) at t in [-1, 1]; shape t.shape + (degree+1,).  Python-float scalars times
    fp32 tensors, in the reference's order of operations (jacobi.py:152-186)."""
    cols = [torch.ones_like(t)]
    if degree > 0:
        cols.append(((alpha + beta + 2) * t + (alpha - beta)) / 2)
        s = alpha + beta
        dsq = alpha ** 2 - beta ** 2
        for n in range(2, degree + 1):
            nf = float(n)
            lead = 2 * nf + s - 1
            inner = (2 * nf + s) * (2 * nf + s - 2) * t + dsq
            k1 = lead * inner
            k2 = -2 * (nf + alpha - 1) * (nf + beta - 1) * (2 * nf + s)
            den = 2 * nf * (nf + s) * (2 * nf + s - 2)
            cols.append((k1 * cols[n - 1] + k2 * cols[n - 2]) / den)
    return torch.stack(cols, dim=-1)


def jacobi_forward(x: torch.Tensor, coeffs: torch.Tensor, alpha: float = 0.0, beta: float = 0.0) -> torch.Tensor:
    x = x.view(-1, coeffs.shape[0])
    phi = jacobi_basis(torch.tanh(x), coeffs.shape[2] - 1, alpha, beta)
    return torch.einsum('bid,iod->bo', phi, coeffs)


# ---------------------------------------------------------------------------------------------------------------
# Hermite
# ---------------------------------------------------------------------------------------------------------------
def hermite_normalize(x: torch.Tensor, domain=None, normalize_domain: bool = True) -> torch.Tensor:
    """hermite.py:85-116: a finite domain with normalisation on maps linearly onto [-3, 3]; otherwise 3 tanh x."""
    if normalize_domain and domain is not None and math.isfinite(domain[0]) and math.isfinite(domain[1]):
        lo, hi = domain
        return (6.0 / (hi - lo)) * (x - lo) - 3.0
    return torch.tanh(x) * 3.0


def hermite_basis(u: torch.Tensor, degree: int, scaling: str = "physicist") -> torch.Tensor:
    """H_0..H_degree (physicist) or He_0..He_degree (probabilist) at u; hermite.py:163-233."""
    if scaling not in ("physicist", "probabilist"):
        raise ValueError(scaling)
    cols = [torch.ones_like(u)]
    if degree > 0:
        if scaling == "physicist":
            cols.append(2 * u)
            for n in range(2, degree + 1):
                cols.append(2 * u * cols[n - 1] - 2 * (n - 1) * cols[n - 2])
        else:
            cols.append(u.clone())     # the reference clones here, which fixes autograd's summation order for dx
            for n in range(2, degree + 1):
                cols.append(u * cols[n - 1] - (n - 1) * cols[n - 2])
    return torch.stack(cols, dim=-1)


def hermite_forward(x: torch.Tensor, coeffs: torch.Tensor, scaling: str = "physicist", domain=None,
                    normalize_domain: bool = True) -> torch.Tensor:
    x = x.view(-1, coeffs.shape[0])
    phi = hermite_basis(hermite_normalize(x, domain, normalize_domain), coeffs.shape[2] - 1, scaling)
    return torch.einsum('bid,iod->bo', phi, coeffs)


# ---------------------------------------------------------------------------------------------------------------
# forward + autograd backward for either family
# ---------------------------------------------------------------------------------------------------------------
def forward(family: dict, x: torch.Tensor, coeffs: torch.Tensor) -> torch.Tensor:
    """`family` is {'kind': 'jacobi', 'alpha': .., 'beta': ..} or {'kind': 'hermite', 'scaling': .., 'domain': ..,
    'normalize_domain': ..}."""
    if family["kind"] == "jacobi":
        return jacobi_forward(x, coeffs, family.get("alpha", 0.0), family.get("beta", 0.0))
    if family["kind"] == "hermite":
        return hermite_forward(x, coeffs, family.get("scaling", "physicist"), family.get("domain"),
                               family.get("normalize_domain", True))
    raise KeyError(family["kind"])


def forward_backward(family: dict, x: torch.Tensor, coeffs: torch.Tensor, dy: torch.Tensor):
    """(y, dC, dx) with dC in the parameter's layout [in, out, deg+1].  At degree 0 the output does not depend on
    x and autograd leaves x.grad unset; dx is returned as zeros then."""
    xr = x.detach().clone().requires_grad_(True)
    cr = coeffs.detach().clone().requires_grad_(True)
    y = forward(family, xr, cr)
    y.backward(dy)
    dx = xr.grad.detach() if xr.grad is not None else torch.zeros_like(x)
    return y.detach(), cr.grad.detach(), dx
