"""CPU restatement of the reference ChebyKAN layer (0xEodum/KAN, version 0.4.0).

TEST INFRASTRUCTURE ONLY: a checker and a timed CPU stand-in.  The shipped
package never imports it and has no CPU fallback.

Parity pin.  The reference holds no tests, golden vectors or known-answer
fixtures for this path.  The pin is therefore the reference itself: in a
container where the reference tree is importable, ``tests/test_oracle.py``
asserts that every function below reproduces the unmodified reference
bit-for-bit on seeded inputs (same ATen CPU kernels, same op order), and
``tests/golden/make_golden.py`` stores outputs of the unmodified reference as
fixtures that travel with the repository.

Every function cites the reference lines it restates (paths inside the
reference project).
"""
from __future__ import annotations

import numpy as np
import torch


# --------------------------------------------------------------------------
# construction                                   kan/layers/chebykan.py:47-51
# --------------------------------------------------------------------------
def init_coeffs(input_dim: int, output_dim: int, degree: int,
                init_scale: float | None = None) -> torch.Tensor:
    """cheby_coeffs[in, out, deg+1] ~ N(0, std) drawn from the global CPU RNG.

    kan/layers/chebykan.py:47  ``init_scale = init_scale or 1/(in*(deg+1))``
    (a falsy 0.0 therefore selects the default) and :48-51 ``torch.empty`` +
    ``nn.init.normal_(mean=0, std=init_scale)``.  ``init_scale`` is a standard
    deviation, not a variance.
    """
    init_scale = init_scale or 1.0 / (input_dim * (degree + 1))
    c = torch.empty(input_dim, output_dim, degree + 1)
    torch.nn.init.normal_(c, mean=0.0, std=init_scale)
    return c


# --------------------------------------------------------------------------
# basis                                         kan/basis/chebyshev.py:68-172
# --------------------------------------------------------------------------
def normalize_input(x: torch.Tensor) -> torch.Tensor:
    """kan/basis/chebyshev.py:78 — t = tanh(x)."""
    return torch.tanh(x)


def basis_closed_form(t: torch.Tensor, degree: int) -> torch.Tensor:
    """Phi[b,i,d] = cos(d * acos(clamp(t,-1,1))), the reference's default path.

    kan/basis/chebyshev.py:130-145: view to [B,in,1], clamp, acos, multiply by
    arange(0..deg) (fp32), cos.
    """
    b, n = t.shape
    t = t.view(b, n, 1)
    theta = torch.acos(torch.clamp(t, -1.0, 1.0))
    arange = torch.arange(0, degree + 1, dtype=torch.float32)
    return torch.cos(theta * arange)


def basis_recurrence(t: torch.Tensor, degree: int) -> torch.Tensor:
    """T_0=1, T_1=t, T_n = 2 t T_{n-1} - T_{n-2}; the reference's opt-in path.

    kan/basis/chebyshev.py:158-172 (in-place slice writes, loop over n).
    """
    b, n = t.shape
    out = torch.ones(b, n, degree + 1, dtype=t.dtype)
    if degree > 0:
        out[:, :, 1] = t
        for k in range(2, degree + 1):
            out[:, :, k] = 2 * t * out[:, :, k - 1] - out[:, :, k - 2]
    return out


def forward(x: torch.Tensor, coeffs: torch.Tensor,
            use_recurrence: bool = False) -> torch.Tensor:
    """y[b,o] = sum_i sum_d coeffs[i,o,d] * T_d(tanh x[b,i]).

    kan/layers/chebykan.py:64 (flatten every leading dimension into rows) and
    kan/basis/chebyshev.py:92-101 (view, tanh, basis, einsum 'bid,iod->bo').
    """
    degree = coeffs.shape[2] - 1
    x = x.view(-1, coeffs.shape[0])
    t = normalize_input(x)
    phi = basis_recurrence(t, degree) if use_recurrence else basis_closed_form(t, degree)
    return torch.einsum('bid,iod->bo', phi, coeffs)


def forward_backward(x: torch.Tensor, coeffs: torch.Tensor, dy: torch.Tensor,
                     use_recurrence: bool = False, need_dx: bool = True):
    """Forward plus the backward PyTorch autograd derives from it.

    The reference has no hand-written backward: gradients are autograd over
    kan/basis/chebyshev.py:78-145.  Returns (y, dC, dx) with dC in the
    parameter's own layout [in, out, deg+1]; dx is None when not requested.
    """
    xr = x.detach().clone().requires_grad_(need_dx)
    cr = coeffs.detach().clone().requires_grad_(True)
    y = forward(xr, cr, use_recurrence)
    y.backward(dy)
    return y.detach(), cr.grad.detach(), (xr.grad.detach() if need_dx else None)


# --------------------------------------------------------------------------
# float64 closed-form truth (independent of autograd); used to show which of
# two fp32 results is nearer the exact value and to check the analytic
# backward identities the CUDA kernels implement.
# --------------------------------------------------------------------------
def analytic_f64(x: np.ndarray, coeffs: np.ndarray, dy: np.ndarray | None = None):
    """fp64 y, dC, dx from the recurrence and its derivative.

    dC[i,o,d] = sum_b T_d(t_bi) dY[b,o]
    dx[b,i]   = (1 - t^2) * sum_d T_d'(t_bi) * sum_o dY[b,o] C[i,o,d]
    with T_d' = d * U_{d-1},  U_0 = 1, U_1 = 2t, U_n = 2 t U_{n-1} - U_{n-2}.
    This is the derivative of kan/basis/chebyshev.py:78-145 wherever |t| < 1.
    """
    x = np.asarray(x, dtype=np.float64)
    c = np.asarray(coeffs, dtype=np.float64)
    n_in, n_out, dp1 = c.shape
    x = x.reshape(-1, n_in)
    t = np.tanh(x)
    T = np.ones(x.shape + (dp1,))
    dT = np.zeros(x.shape + (dp1,))
    if dp1 > 1:
        T[..., 1] = t
        U_prev, U_cur = np.ones_like(t), 2 * t  # U_0, U_1
        dT[..., 1] = 1.0
        for k in range(2, dp1):
            T[..., k] = 2 * t * T[..., k - 1] - T[..., k - 2]
            dT[..., k] = k * U_cur
            U_prev, U_cur = U_cur, 2 * t * U_cur - U_prev
    y = np.einsum('bid,iod->bo', T, c)
    if dy is None:
        return y, None, None
    dy = np.asarray(dy, dtype=np.float64)
    dC = np.einsum('bid,bo->iod', T, dy)
    G = np.einsum('bo,iod->bid', dy, c)
    dx = (1 - t * t) * (dT * G).sum(-1)
    return y, dC, dx


def rel_l2(a, b) -> float:
    """||a - b||_2 / ||b||_2 over the whole tensor, accumulated in fp64."""
    a = torch.as_tensor(a).detach().double().cpu().reshape(-1)
    b = torch.as_tensor(b).detach().double().cpu().reshape(-1)
    den = float(torch.linalg.vector_norm(b))
    num = float(torch.linalg.vector_norm(a - b))
    if den == 0.0:
        return 0.0 if num == 0.0 else float('inf')
    return num / den


# --------------------------------------------------------------------------
# optimizers — third-party torch.optim as called by the reference's README
# training loop (README.md:59-66): Adam(lr) with default betas/eps and plain
# SGD(lr).  Restated so that the update can be checked without torch.optim.
# --------------------------------------------------------------------------
def sgd_step(p: torch.Tensor, g: torch.Tensor, lr: float) -> torch.Tensor:
    return p - lr * g


def adam_step(p, g, m, v, step: int, lr: float, b1=0.9, b2=0.999, eps=1e-8):
    """One torch.optim.Adam update (no weight decay, no amsgrad)."""
    m = b1 * m + (1 - b1) * g
    v = b2 * v + (1 - b2) * g * g
    bc1 = 1 - b1 ** step
    bc2 = 1 - b2 ** step
    denom = v.sqrt() / (bc2 ** 0.5) + eps
    p = p - (lr / bc1) * m / denom
    return p, m, v
