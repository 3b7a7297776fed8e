"""Drop-in JacobiKANLayer and HermiteKANLayer on the sm_100a kernels.

The reference's Jacobi and Hermite layers (kan/layers/jacobikan.py:10-113, kan/layers/hermitekan.py:10-121)
have the Chebyshev layer's structure - normalise the input, evaluate a three-term recurrence, contract with
``coefficients[in, out, deg+1]`` through ``einsum('bid,iod->bo')`` - so they run on the same fused kernels
with the recurrence coefficients swapped (the library's ``chebykan_family_*`` entry points).  Constructors,
parameter names (``jacobi_coeffs`` / ``hermite_coeffs``), RNG consumption, ``state_dict``, ``forward``'s flatten
rule, ``get_coefficients``, ``get_analytical_form`` and ``extra_repr`` mirror the reference.  ``math_mode='fp32'``
(default) runs forward, dC and dx on the FFMA pipe with a correctly rounded tanh (rel-L2 <= 1e-5 to the reference);
``'tf32'`` / ``'bf16'`` run forward and backward on the tcgen05 tensor cores (rel-L2 <= 2e-3; the backward
contracts in tf32 in both).
There is no CPU path.
"""
from __future__ import annotations

import math
from typing import Any, Dict, Optional, Tuple

import torch
import torch.nn as nn

from . import ops
from .layer import KANLayer, _PackedCache, _aligned


# ---------------------------------------------------------------------------------------------------------------
# stand-ins for the reference's basis objects (used when the reference package is not importable)
# ---------------------------------------------------------------------------------------------------------------
class JacobiBasis:
    """Descriptor of the Jacobi basis P_d^(alpha,beta) on tanh(x) (kan/basis/jacobi.py:9-120)."""

    def __init__(self, degree: int, alpha: float = 0.0, beta: float = 0.0, domain: Tuple[float, float] = (-1, 1)):
        if alpha <= -1 or beta <= -1:
            raise ValueError(f"Parameters must satisfy α, β > -1, got α={alpha}, β={beta}")
        self.degree = degree
        self.alpha = alpha
        self.beta = beta
        self._domain = domain
        self.arange = torch.arange(0, degree + 1, dtype=torch.float32)

    @property
    def name(self) -> str:
        return f"Jacobi-{self.degree}-{self.alpha}-{self.beta}"

    @property
    def domain(self) -> Tuple[float, float]:
        return self._domain

    def normalize_input(self, x: torch.Tensor) -> torch.Tensor:
        return ops.family_normalize(family_of(self), _aligned(x))

    def basis_functions(self, x: torch.Tensor) -> torch.Tensor:
        """P_0..P_degree at normalised points: shape x.shape + (degree+1,)  (kan/basis/jacobi.py:122-188)."""
        return ops.family_basis(family_of(self), _aligned(x), self.degree)

    def forward(self, x: torch.Tensor, coefficients: torch.Tensor) -> torch.Tensor:
        return family_apply(x.view(-1, coefficients.shape[0]), coefficients, family_of(self), None)


class HermiteBasis:
    """Descriptor of the Hermite basis (physicist's H_d or probabilist's He_d) on 3 tanh(x), or on the affine
    image of a finite domain in [-3, 3] (kan/basis/hermite.py:8-141)."""

    def __init__(self, degree: int, scaling: str = 'physicist', domain: Optional[Tuple[float, float]] = None,
                 normalize_domain: bool = True):
        if scaling not in ['physicist', 'probabilist']:
            raise ValueError(f"Invalid scaling: {scaling}. Must be one of ['physicist', 'probabilist']")
        self.degree = degree
        self.scaling = scaling
        self._normalize_domain = normalize_domain
        self._domain = domain or (-float('inf'), float('inf'))
        self.arange = torch.arange(0, degree + 1, dtype=torch.float32)

    @property
    def name(self) -> str:
        return f"Hermite-{self.degree}-{self.scaling}"

    @property
    def domain(self) -> Tuple[float, float]:
        return self._domain

    def normalize_input(self, x: torch.Tensor) -> torch.Tensor:
        return ops.family_normalize(family_of(self), _aligned(x))

    def basis_functions(self, x: torch.Tensor) -> torch.Tensor:
        """H_0..H_degree (or He) at normalised points: shape x.shape + (degree+1,)  (kan/basis/hermite.py:143-233)."""
        return ops.family_basis(family_of(self), _aligned(x), self.degree)

    def forward(self, x: torch.Tensor, coefficients: torch.Tensor) -> torch.Tensor:
        return family_apply(x.view(-1, coefficients.shape[0]), coefficients, family_of(self), None)


def family_of(basis):
    """The library's description of a basis object: works on the stand-ins above and on the reference's own
    JacobiBasis / HermiteBasis, which carry the same attributes."""
    if hasattr(basis, "alpha") and hasattr(basis, "beta"):
        return ops.make_family("jacobi", alpha=basis.alpha, beta=basis.beta)
    if hasattr(basis, "scaling"):
        kind = "hermite" if basis.scaling == "physicist" else "hermite_prob"
        lo, hi = basis._domain
        if basis._normalize_domain and math.isfinite(lo) and math.isfinite(hi):
            # kan/basis/hermite.py:102-112: scale * (x - domain_min) - 3 with scale = 6 / (max - min)
            return ops.make_family(kind, scale=6.0 / (hi - lo), affine=True, shift=lo, offset=-3.0)
        return ops.make_family(kind, scale=3.0)
    raise TypeError(f"no sm_100a kernels for basis {type(basis).__name__}")


# ---------------------------------------------------------------------------------------------------------------
# autograd glue
# ---------------------------------------------------------------------------------------------------------------
class _FamilyKANFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, coeffs, family, cache, mode):
        n_in, n_out, dp1 = coeffs.shape
        packed = cache.get(coeffs, mode) if cache is not None else ops.pack_coeffs(coeffs.detach(), mode)
        x = _aligned(x)
        y = ops.family_forward(family, x, packed, n_in, n_out, dp1 - 1, mode)
        ctx.save_for_backward(x, coeffs)
        ctx.family = family
        ctx.mode = mode
        return y

    @staticmethod
    def backward(ctx, dy):
        x, coeffs = ctx.saved_tensors
        n_in, n_out, dp1 = coeffs.shape
        dy = _aligned(dy)
        dx = dc = None
        if ctx.needs_input_grad[1]:
            dc = ops.family_bwd_dcoeff(ctx.family, x, dy, n_in, n_out, dp1 - 1, ctx.mode)
        if ctx.needs_input_grad[0]:
            dx = ops.family_bwd_dx(ctx.family, x, dy, _aligned(coeffs.detach()), ctx.mode)
        return dx, dc, None, None, None


def family_apply(x: torch.Tensor, coeffs: torch.Tensor, family, cache=None, mode: str = "fp32") -> torch.Tensor:
    """y = sum_i sum_d coeffs[i,o,d] P_d(u(x[b,i])) with autograd, x already [B, in]."""
    if not x.is_cuda or not coeffs.is_cuda:
        raise RuntimeError("kan_b200 layers run on CUDA (sm_100a) only: move the layer and its input to the GPU; "
                           "there is no CPU path")
    if x.device != coeffs.device:
        raise RuntimeError(f"input is on {x.device} but the layer's coefficients are on {coeffs.device}")
    if x.dtype != torch.float32:
        raise RuntimeError(f"expected scalar type Float but found {str(x.dtype).replace('torch.', '').capitalize()}")
    return _FamilyKANFunction.apply(x, coeffs, family, cache, mode)


# ---------------------------------------------------------------------------------------------------------------
# the layers
# ---------------------------------------------------------------------------------------------------------------
FAMILY_MODES = ("fp32", "tf32", "bf16")


def _check_mode(math_mode: str) -> None:
    if math_mode not in FAMILY_MODES:
        raise ValueError(f"math_mode must be one of {list(FAMILY_MODES)} for this layer, got {math_mode!r}")


def make_jacobikan_layer_class(base_cls, basis_cls, name: str = "JacobiKANLayer"):
    """JacobiKANLayer on a given (KANLayer base, JacobiBasis) pair: the stand-ins, or the reference's own classes."""

    class _Layer(base_cls):
        """KAN layer on Jacobi polynomials, computed by sm_100a CUDA kernels.
        Args as in the reference (kan/layers/jacobikan.py:20-33): input_dim, output_dim, degree, alpha, beta, init_scale;
        keyword-only math_mode: 'fp32' (default), 'tf32' or 'bf16' (tensor cores)."""

        def __init__(self, input_dim: int, output_dim: int, degree: int, alpha: float = 0.0, beta: float = 0.0,
                     init_scale: float = None, *, math_mode: str = "fp32"):
            _check_mode(math_mode)
            if alpha <= -1 or beta <= -1:
                raise ValueError(f"Parameters must satisfy α, β > -1, got α={alpha}, β={beta}")
            basis_function = basis_cls(degree=degree, alpha=alpha, beta=beta)
            super().__init__(input_dim=input_dim, output_dim=output_dim, basis_function=basis_function)
            self.degree = degree
            self.math_mode = math_mode
            self.alpha = alpha
            self.beta = beta
            # identical RNG consumption to kan/layers/jacobikan.py:58-63
            init_scale = init_scale or 1.0 / (input_dim * (degree + 1))
            self.jacobi_coeffs = nn.Parameter(torch.empty(input_dim, output_dim, degree + 1))
            nn.init.normal_(self.jacobi_coeffs, mean=0.0, std=init_scale)
            self._packed = _PackedCache()
            self._family = family_of(basis_function)

        def forward(self, x: torch.Tensor) -> torch.Tensor:
            x = x.view(-1, self.input_dim)
            return family_apply(x, self.jacobi_coeffs, self._family, self._packed, self.math_mode)

        def get_analytical_form(self) -> Dict[str, Any]:
            return {
                'type': 'JacobiKANLayer',
                'input_dim': self.input_dim,
                'output_dim': self.output_dim,
                'degree': self.degree,
                'alpha': self.alpha,
                'beta': self.beta,
                'basis': self.basis_function.name,
                'coefficients': self.jacobi_coeffs.detach().cpu().numpy(),
            }

        def get_coefficients(self) -> torch.Tensor:
            return self.jacobi_coeffs

        def extra_repr(self) -> str:
            return (f'input_dim={self.input_dim}, output_dim={self.output_dim}, degree={self.degree}, '
                    f'alpha={self.alpha}, beta={self.beta}')

        def _apply(self, fn, *args, **kwargs):
            self._packed.clear()
            return super()._apply(fn, *args, **kwargs)

    _Layer.__name__ = name
    _Layer.__qualname__ = name
    return _Layer


def make_hermitekan_layer_class(base_cls, basis_cls, name: str = "HermiteKANLayer"):
    """HermiteKANLayer on a given (KANLayer base, HermiteBasis) pair."""

    class _Layer(base_cls):
        """KAN layer on Hermite polynomials, computed by sm_100a CUDA kernels.
        Args as in the reference (kan/layers/hermitekan.py:22-40): input_dim, output_dim, degree, scaling, domain,
        normalize_domain, init_scale; keyword-only math_mode: 'fp32' (default), 'tf32' or 'bf16' (tensor cores)."""

        def __init__(self, input_dim: int, output_dim: int, degree: int, scaling: str = 'physicist',
                     domain: Optional[Tuple[float, float]] = None, normalize_domain: bool = True,
                     init_scale: float = None, *, math_mode: str = "fp32"):
            _check_mode(math_mode)
            basis_function = basis_cls(degree=degree, scaling=scaling, domain=domain,
                                       normalize_domain=normalize_domain)
            super().__init__(input_dim=input_dim, output_dim=output_dim, basis_function=basis_function)
            self.degree = degree
            self.math_mode = math_mode
            self.scaling = scaling
            self.domain = domain
            self.normalize_domain = normalize_domain
            # identical RNG consumption to kan/layers/hermitekan.py:60-65
            init_scale = init_scale or 1.0 / (input_dim * (degree + 1))
            self.hermite_coeffs = nn.Parameter(torch.empty(input_dim, output_dim, degree + 1))
            nn.init.normal_(self.hermite_coeffs, mean=0.0, std=init_scale)
            self._packed = _PackedCache()
            self._family = family_of(basis_function)

        def forward(self, x: torch.Tensor) -> torch.Tensor:
            x = x.view(-1, self.input_dim)
            return family_apply(x, self.hermite_coeffs, self._family, self._packed, self.math_mode)

        def get_analytical_form(self) -> Dict[str, Any]:
            return {
                'type': 'HermiteKANLayer',
                'input_dim': self.input_dim,
                'output_dim': self.output_dim,
                'degree': self.degree,
                'scaling': self.scaling,
                'domain': self.domain,
                'normalize_domain': self.normalize_domain,
                'basis': self.basis_function.name,
                'coefficients': self.hermite_coeffs.detach().cpu().numpy(),
            }

        def get_coefficients(self) -> torch.Tensor:
            return self.hermite_coeffs

        def extra_repr(self) -> str:
            domain_str = f", domain={self.domain}" if self.domain else ""
            normalize_str = f", normalize_domain={self.normalize_domain}"
            return (f'input_dim={self.input_dim}, output_dim={self.output_dim}, '
                    f'degree={self.degree}, scaling={self.scaling}{domain_str}{normalize_str}')

        def _apply(self, fn, *args, **kwargs):
            self._packed.clear()
            return super()._apply(fn, *args, **kwargs)

    _Layer.__name__ = name
    _Layer.__qualname__ = name
    return _Layer


JacobiKANLayer = make_jacobikan_layer_class(KANLayer, JacobiBasis)
HermiteKANLayer = make_hermitekan_layer_class(KANLayer, HermiteBasis)


def install_into_reference():
    """Swap both layers into an importable reference package: ``kan.layers.LAYER_REGISTRY['jacobikan' / 'hermitekan']``
    (kan/layers/__init__.py:18-27), ``kan.layers.JacobiKANLayer / HermiteKANLayer`` and the same names on ``kan``,
    built on the reference's own ``KANLayer`` and basis classes.  Returns (JacobiKANLayer, HermiteKANLayer)."""
    import kan  # the reference package; raises ImportError when absent
    from kan.layers.base import KANLayer as RefKANLayer
    from kan.basis.jacobi import JacobiBasis as RefJacobi
    from kan.basis.hermite import HermiteBasis as RefHermite
    jac = make_jacobikan_layer_class(RefKANLayer, RefJacobi)
    her = make_hermitekan_layer_class(RefKANLayer, RefHermite)
    kan.layers.LAYER_REGISTRY['jacobikan'] = jac
    kan.layers.LAYER_REGISTRY['hermitekan'] = her
    kan.layers.JacobiKANLayer = jac
    kan.layers.HermiteKANLayer = her
    if hasattr(kan, "JacobiKANLayer"):
        kan.JacobiKANLayer = jac
    if hasattr(kan, "HermiteKANLayer"):
        kan.HermiteKANLayer = her
    return jac, her
