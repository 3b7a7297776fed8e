"""Mean-squared-error loss computed together with its gradient.

``nn.MSELoss()(model(x), target)`` as the reference's training loop writes it
(README.md:57-69) costs three passes over the output in torch: square into a
temporary, average, and on the way back re-read output and target to form the
gradient.  ``mse_loss`` reads output and target once, writes the gradient and
the scalar loss in that pass (``chebykan_mse_loss_grad``), and hands the stored
gradient to autograd in backward.  Same value and gradient as torch's, mean
reduction only.
"""
from __future__ import annotations

import torch

from . import ops


class _MSELossFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y, target, n_mean):
        y = y.contiguous()
        target = target.contiguous()
        loss, dy = ops.mse_loss_grad(y, target, n_mean)
        ctx.save_for_backward(dy)
        return loss

    @staticmethod
    def backward(ctx, grad_loss):
        (dy,) = ctx.saved_tensors
        # chain rule: multiply by the incoming scalar; the kernel leaves dy alone when it is exactly 1
        # (loss.backward() itself), so the usual step pays for no second pass
        g = grad_loss.detach().to(torch.float32).contiguous().view(1)
        ops.scale_by_device_scalar(dy, g)
        return dy, None, None


def mse_loss(y: torch.Tensor, target: torch.Tensor, n_mean: int | None = None) -> torch.Tensor:
    """mean((y - target)^2) with the gradient prepared in the same pass.

    ``n_mean`` overrides the divisor (the element count of the global batch when the rows are sharded
    over several GPUs, so that summing the ranks' gradients gives the single-GPU gradient).  Gradients
    flow to ``y`` only.  The stored gradient is consumed by the first backward: do not call backward
    twice on the same loss (``retain_graph`` is not supported)."""
    if not y.is_cuda or not target.is_cuda:
        raise RuntimeError("kan_b200.mse_loss runs on CUDA only")
    if target.requires_grad:
        raise RuntimeError("kan_b200.mse_loss does not differentiate with respect to the target")
    return _MSELossFunction.apply(y, target, n_mean)


class MSELoss(torch.nn.Module):
    """Module form of ``mse_loss`` (mean reduction), usable wherever ``nn.MSELoss()`` stands."""

    def __init__(self, n_mean: int | None = None):
        super().__init__()
        self.n_mean = n_mean

    def forward(self, y: torch.Tensor, target: torch.Tensor) -> torch.Tensor:
        return mse_loss(y, target, self.n_mean)
