"""kan_b200 — the ChebyKAN layer hot path of 0xEodum/KAN on NVIDIA B200 (sm_100a).

Public surface: ``ChebyKANLayer`` (drop-in for kan.layers.chebykan.ChebyKANLayer),
``install_into_reference`` (swap it into the reference's layer registry), ``JacobiKANLayer`` and
``HermiteKANLayer`` (the reference's other recurrence-based layers on the same fp32 kernels), the
functional ``ops``, the kernel-backed ``optim.SGD`` / ``optim.Adam`` and the
data-parallel helpers in ``dp``.  Everything computes in hand-written CUDA
behind the C ABI of ``include/chebykan_b200.h``; there is no CPU fallback.
"""
from .layer import ChebyKANLayer, ChebyshevBasis, KANLayer, chebykan_apply, install_into_reference
from .poly import HermiteBasis, HermiteKANLayer, JacobiBasis, JacobiKANLayer
from .stack import FusedChebyKANStack, fuse_layernorm
from .loss import MSELoss, mse_loss
from . import ops, optim, dp, workloads, graph, poly, small

__all__ = ["MSELoss", "mse_loss", "FusedChebyKANStack", "fuse_layernorm", "ChebyKANLayer", "ChebyshevBasis", "KANLayer",
           "JacobiKANLayer", "HermiteKANLayer", "JacobiBasis", "HermiteBasis", "chebykan_apply", "install_into_reference",
           "ops", "optim", "dp", "workloads", "graph", "poly", "small"]
__version__ = "0.1.0"
