"""Drop-in ChebyKANLayer backed by the sm_100a kernels.

Mirrors the reference's ``kan.layers.chebykan.ChebyKANLayer``
(kan/layers/chebykan.py:10-101): same constructor, the same parameter
``cheby_coeffs[in, out, deg+1]`` drawn from the global CPU RNG in the same
way, the same ``state_dict``, ``forward`` flatten rule, ``get_coefficients``,
``get_analytical_form`` and ``extra_repr``.  ``forward`` and its autograd
backward run hand-written CUDA through the C ABI; there is no CPU path and no
PyTorch fallback: a CPU input raises.
"""
from __future__ import annotations

from abc import ABC, abstractmethod
from typing import Any, Dict, Tuple

import torch
import torch.nn as nn

from . import ops


# ---------------------------------------------------------------------------
# local stand-ins for the reference's abstract bases, used when the reference
# package is not importable (kan/layers/base.py:11-141, kan/basis/base.py:7-94,
# kan/basis/chebyshev.py:24-66)
# ---------------------------------------------------------------------------
class KANLayer(nn.Module, ABC):
    """Same abstract surface as the reference's kan.layers.base.KANLayer."""

    @abstractmethod
    def __init__(self, input_dim: int, output_dim: int, basis_function, **kwargs):
        super().__init__()
        self.input_dim = input_dim
        self.output_dim = output_dim
        self.basis_function = basis_function

    @abstractmethod
    def forward(self, x: torch.Tensor) -> torch.Tensor: ...

    @property
    def basis(self):
        return self.basis_function

    @abstractmethod
    def get_analytical_form(self) -> Dict[str, Any]: ...

    @abstractmethod
    def get_coefficients(self) -> torch.Tensor: ...


class ChebyshevBasis:
    """Descriptor of the Chebyshev basis (degree, name, domain).

    Carries the attributes the reference's ChebyshevBasis exposes
    (kan/basis/chebyshev.py:24-66).  ``forward`` evaluates the expansion with
    the fused CUDA kernel; the [B, in, deg+1] basis tensor is never built.
    """

    def __init__(self, degree: int, domain: Tuple[float, float] = (-1, 1), use_recurrence: bool = False):
        self.degree = degree
        self._domain = domain
        self.use_recurrence = use_recurrence
        self.arange = torch.arange(0, degree + 1, dtype=torch.float32)

    @property
    def name(self) -> str:
        return f"Chebyshev-{self.degree}"

    @property
    def domain(self) -> Tuple[float, float]:
        return self._domain

    def forward(self, x: torch.Tensor, coefficients: torch.Tensor) -> torch.Tensor:
        x = x.view(-1, coefficients.shape[0])
        return chebykan_apply(x, coefficients, "fp32", None)

    def normalize_input(self, x: torch.Tensor) -> torch.Tensor:
        """t = tanh(x) (kan/basis/chebyshev.py:68-78)."""
        return ops.normalize_input(_aligned(x))

    def basis_functions(self, x: torch.Tensor) -> torch.Tensor:
        """T_0..T_degree at normalised points x in [-1, 1]: shape x.shape + (degree+1,)
        (kan/basis/chebyshev.py:103-172; both of the reference's evaluation paths give these values)."""
        return ops.basis_functions(_aligned(x), self.degree)

    def derivative(self, x: torch.Tensor, coefficients: torch.Tensor, order: int = 1) -> torch.Tensor:
        """d/dx of the expansion summed over the inputs, shape (batch, output_dim); order 0 is ``forward``.

        The reference's method of this name (kan/basis/chebyshev.py:174-267) does not return a derivative of the
        expansion (its coefficient rule is wrong and it re-applies tanh); this one returns the values autograd
        gives for sum_i d y_o / d x_i.  Orders above 1 are not implemented."""
        if order == 0:
            return self.forward(x, coefficients)
        if order != 1:
            raise NotImplementedError("only first derivatives are implemented")
        x = _aligned(x.view(-1, coefficients.shape[0]))
        return ops.jacobian(x, _aligned(coefficients.detach())).sum(-1)


# ---------------------------------------------------------------------------
# autograd glue
# ---------------------------------------------------------------------------
class _PackedCache:
    """Packed coefficient buffers, one per math mode, rebuilt when the parameter changes."""

    def __init__(self):
        self._entries = {}

    def get(self, coeffs: torch.Tensor, mode: str) -> torch.Tensor:
        key = (coeffs.data_ptr(), coeffs._version, tuple(coeffs.shape))
        ent = self._entries.get(mode)
        if ent is None or ent[0] != key:
            buf = ent[1] if ent is not None and ent[1].device == coeffs.device else None
            try:
                buf = ops.pack_coeffs(coeffs.detach(), mode, out=buf)
            except RuntimeError:
                buf = ops.pack_coeffs(coeffs.detach(), mode)
            self._entries[mode] = (key, buf)
            ent = self._entries[mode]
        return ent[1]

    def clear(self):
        self._entries.clear()


def _aligned(t: torch.Tensor) -> torch.Tensor:
    """Contiguous and 16-byte aligned (a view into the middle of a buffer may be neither): the kernels use
    vector and TMA accesses.  Fresh torch allocations are always aligned, so a copy fixes both."""
    t = t.contiguous()
    if t.numel() and t.data_ptr() % 16:
        t = t.clone()
    return t


class _ChebyKANFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, coeffs, mode, cache):
        n_in, n_out, dp1 = coeffs.shape
        packed = cache.get(coeffs, mode) if cache is not None else ops.pack_coeffs(coeffs.detach(), mode)
        x = _aligned(x)
        y = ops.forward(x, packed, n_in, n_out, dp1 - 1, mode)
        ctx.save_for_backward(x, coeffs)
        ctx.mode = mode
        return y

    @staticmethod
    def backward(ctx, dy):
        x, coeffs = ctx.saved_tensors
        n_in, n_out, dp1 = coeffs.shape
        dy = _aligned(dy)
        dx = dc = None
        if ctx.needs_input_grad[1]:
            dc = ops.bwd_dcoeff(x, dy, n_in, n_out, dp1 - 1, ctx.mode)
        if ctx.needs_input_grad[0]:
            dx = ops.bwd_dx(x, dy, coeffs.detach(), ctx.mode)
        return dx, dc, None, None


def chebykan_apply(x: torch.Tensor, coeffs: torch.Tensor, mode: str = "fp32", cache=None) -> torch.Tensor:
    """y = sum_i sum_d coeffs[i,o,d] T_d(tanh x[b,i]) with autograd, x already [B, in]."""
    if not x.is_cuda or not coeffs.is_cuda:
        raise RuntimeError("kan_b200.ChebyKANLayer runs on CUDA (sm_100a) only: move the layer and its "
                           "input to the GPU; there is no CPU path")
    if x.device != coeffs.device:
        raise RuntimeError(f"input is on {x.device} but the layer's coefficients are on {coeffs.device}")
    if x.dtype != torch.float32:
        # the reference's einsum raises the same way on a dtype mismatch
        raise RuntimeError(f"expected scalar type Float but found {str(x.dtype).replace('torch.', '').capitalize()}")
    return _ChebyKANFunction.apply(x, coeffs, mode, cache)


# ---------------------------------------------------------------------------
# the layer
# ---------------------------------------------------------------------------
def make_chebykan_layer_class(base_cls, basis_cls, name: str = "ChebyKANLayer"):
    """Build the layer class on a given (KANLayer base, ChebyshevBasis) pair.

    Called once with the local stand-ins, and by ``install_into_reference``
    with the reference's own classes so that ``isinstance(layer, kan.KANLayer)``
    and ``isinstance(layer.basis_function, kan.ChebyshevBasis)`` hold.
    """

    class _Layer(base_cls):
        __doc__ = ChebyKANLayerDoc

        def __init__(self, input_dim: int, output_dim: int, degree: int,
                     use_recurrence: bool = False, init_scale: float = None, *,
                     math_mode: str = "fp32"):
            if math_mode not in ops.MODES:
                raise ValueError(f"math_mode must be one of {sorted(ops.MODES)}")
            basis_function = basis_cls(degree=degree, use_recurrence=use_recurrence)
            super().__init__(input_dim=input_dim, output_dim=output_dim, basis_function=basis_function)
            self.degree = degree
            self.math_mode = math_mode
            # identical RNG consumption to kan/layers/chebykan.py:47-51
            init_scale = init_scale or 1.0 / (input_dim * (degree + 1))
            self.cheby_coeffs = nn.Parameter(torch.empty(input_dim, output_dim, degree + 1))
            nn.init.normal_(self.cheby_coeffs, mean=0.0, std=init_scale)
            self._packed = _PackedCache()

        def forward(self, x: torch.Tensor) -> torch.Tensor:
            x = x.view(-1, self.input_dim)   # kan/layers/chebykan.py:64
            return chebykan_apply(x, self.cheby_coeffs, self.math_mode, self._packed)

        @torch.no_grad()
        def forward_host(self, x_host: torch.Tensor, out: torch.Tensor = None, chunk_rows: int = 8192) -> torch.Tensor:
            """Inference with HOST tensors in and out, copies overlapped with compute.

            The batch is cut into blocks of `chunk_rows` rows; block k+1 is copied to the GPU
            while block k is computed and block k-1 is copied back (the library's two copy
            streams plus the current stream), so the two directions of the PCIe link work at the
            same time.  `x_host` and `out` should be pinned (the copies are synchronous otherwise);
            returns `out` ([rows, output_dim], pinned if it had to be allocated) after all work
            has finished.
            """
            if x_host.is_cuda:
                raise RuntimeError("forward_host takes a host tensor; call the layer itself for CUDA tensors")
            if x_host.dtype != torch.float32:
                raise RuntimeError(f"expected scalar type Float but found {str(x_host.dtype).replace('torch.', '').capitalize()}")
            dev = self.cheby_coeffs.device
            if dev.type != "cuda":
                raise RuntimeError("move the layer to a CUDA device first")
            packed = self._packed.get(self.cheby_coeffs, self.math_mode)
            out, scratch = ops.forward_host_packed(x_host, packed, self.input_dim, self.output_dim, self.degree,
                                                   self.math_mode, out=out, chunk_rows=chunk_rows,
                                                   scratch=self.__dict__.get("_host_scratch"))
            self.__dict__["_host_scratch"] = scratch
            return out

        @torch.no_grad()
        def jacobian(self, x: torch.Tensor) -> torch.Tensor:
            """True Jacobian d y / d x, shape (batch, output_dim, input_dim), as autograd would give it.

            The reference's ``KANLayer.jacobian`` (kan/layers/base.py:116-141) has this shape but is built
            on ``ChebyshevBasis.derivative``, which is not the derivative of the layer.
            """
            x = _aligned(x.view(-1, self.input_dim))
            if not x.is_cuda:
                raise RuntimeError("kan_b200 runs on CUDA only")
            return ops.jacobian(x, self.cheby_coeffs.detach())

        @torch.no_grad()
        def compute_derivatives(self, x: torch.Tensor, order: int = 1) -> torch.Tensor:
            """First derivative summed over the inputs, shape (batch, output_dim): sum_i d y_o / d x_i.
            Same shape as the reference's ``compute_derivatives`` (kan/layers/base.py:102-114), true values."""
            if order != 1:
                raise NotImplementedError("only first derivatives are implemented")
            return self.jacobian(x).sum(-1)

        def get_analytical_form(self) -> Dict[str, Any]:
            return {
                'type': 'ChebyKANLayer',
                'input_dim': self.input_dim,
                'output_dim': self.output_dim,
                'degree': self.degree,
                'basis': self.basis_function.name,
                'coefficients': self.cheby_coeffs.detach().cpu().numpy(),
            }

        def get_coefficients(self) -> torch.Tensor:
            return self.cheby_coeffs

        def extra_repr(self) -> str:
            return f'input_dim={self.input_dim}, output_dim={self.output_dim}, degree={self.degree}'

        def _apply(self, fn, *args, **kwargs):
            self._packed.clear()
            self.__dict__["_host_pipe"] = None
            return super()._apply(fn, *args, **kwargs)

    _Layer.__name__ = name
    _Layer.__qualname__ = name
    return _Layer


ChebyKANLayerDoc = """KAN layer on Chebyshev polynomials, computed by sm_100a CUDA kernels.

    Args (as in the reference, kan/layers/chebykan.py:21-32):
        input_dim, output_dim, degree, use_recurrence, init_scale
    Keyword-only:
        math_mode: 'fp32' (FFMA, rel-L2 <= 1e-5 to the reference), 'fp32x3' (the same
                   tolerance on the tensor cores: three tf32 products of head/tail
                   splits, forward and - for large layers - backward), 'tf32' or 'bf16'
                   (tcgen05 tensor cores, rel-L2 <= 2e-3).
    ``use_recurrence`` is kept for API compatibility; the kernels always use
    the three-term recurrence, which agrees with the reference's closed form
    to about 1e-6.
"""

ChebyKANLayer = make_chebykan_layer_class(KANLayer, ChebyshevBasis)


def install_into_reference():
    """Swap this layer into an importable reference package.

    Builds the layer on the reference's own ``KANLayer`` / ``ChebyshevBasis``
    and assigns it to ``kan.layers.LAYER_REGISTRY['chebykan']``
    (kan/layers/__init__.py:18-27), ``kan.layers.ChebyKANLayer`` and
    ``kan.ChebyKANLayer``.  The name inside the module ``kan.layers.chebykan``
    is left alone: the reference class refers to itself through it in its own
    ``super()`` call.  Returns the new class.
    """
    import kan  # the reference package; raises ImportError when absent
    from kan.layers.base import KANLayer as RefKANLayer
    from kan.basis.chebyshev import ChebyshevBasis as RefBasis
    cls = make_chebykan_layer_class(RefKANLayer, RefBasis)
    kan.layers.LAYER_REGISTRY['chebykan'] = cls
    kan.layers.ChebyKANLayer = cls
    kan.ChebyKANLayer = cls
    return cls
