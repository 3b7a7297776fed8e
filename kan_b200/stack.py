"""Inference over a stack of ChebyKAN layers with the LayerNorms between them fused away.

The reference chains layers and ``torch.nn.LayerNorm`` modules in a Sequential
(kan/layers/base.py:144-153); every LayerNorm then reads and rewrites the whole
activation.  ``fuse_layernorm`` keeps the same modules and parameters but runs
them differently: layer k's kernel also accumulates each output row's sum and
sum of squares, and layer k+1's kernel normalises the rows while it loads them
(chebykan_fwd_ln), so the activation between two layers is written once and read
once.  Inference only (no autograd); tensor-core math modes only; anything that
does not match the pattern runs through the original modules unchanged.
"""
from __future__ import annotations

from typing import List

import torch
import torch.nn as nn

from . import ops


def _is_cheby(m) -> bool:
    return hasattr(m, "cheby_coeffs") and hasattr(m, "math_mode") and hasattr(m, "_packed")


class FusedChebyKANStack(nn.Module):
    def __init__(self, modules: List[nn.Module]):
        super().__init__()
        self.layers = nn.ModuleList(modules)     # shares the original modules and their parameters

    def _fusable(self, k: int) -> bool:
        """modules[k] is a LayerNorm between two tensor-core ChebyKAN layers of matching width."""
        m = self.layers
        if not (0 < k < len(m) - 1 and isinstance(m[k], nn.LayerNorm)):
            return False
        a, b = m[k - 1], m[k + 1]
        if not (_is_cheby(a) and _is_cheby(b)):
            return False
        if a.math_mode in ("fp32", "fp32x3") or b.math_mode in ("fp32", "fp32x3"):
            return False
        return tuple(m[k].normalized_shape) == (a.output_dim,) and b.input_dim == a.output_dim

    @torch.no_grad()
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        m = self.layers
        k = 0
        ln_in = None          # (stats, gamma, beta, eps) pending for the next ChebyKAN layer
        while k < len(m):
            mod = m[k]
            if _is_cheby(mod):
                x = x.view(-1, mod.input_dim)
                if not x.is_cuda:
                    raise RuntimeError("kan_b200 runs on CUDA only")
                fuse_next = self._fusable(k + 1)
                if ln_in is None and not fuse_next:
                    x = mod(x)
                else:
                    x = x.contiguous()
                    stats_out = torch.zeros(x.shape[0], 2, device=x.device) if fuse_next else None
                    packed = mod._packed.get(mod.cheby_coeffs, mod.math_mode)
                    x = ops.forward_ln(x, packed, mod.input_dim, mod.output_dim, mod.degree, mod.math_mode,
                                       ln_in=ln_in, stats_out=stats_out)
                    ln_in = None
                    if fuse_next:
                        ln = m[k + 1]
                        dev = x.device
                        gamma = ln.weight if ln.weight is not None else torch.ones(mod.output_dim, device=dev)
                        beta = ln.bias if ln.bias is not None else torch.zeros(mod.output_dim, device=dev)
                        ln_in = (stats_out, gamma.detach().contiguous(), beta.detach().contiguous(), ln.eps)
                        k += 1       # the LayerNorm module itself is skipped
            else:
                x = mod(x)
            k += 1
        return x


def fuse_layernorm(model: nn.Sequential) -> FusedChebyKANStack:
    """Wrap a Sequential of ChebyKAN layers and LayerNorms for fused inference (parameters are shared)."""
    return FusedChebyKANStack(list(model.children()))
