"""One-launch training step for a single small ChebyKAN layer.

The reference's own example (README.md:57-69) fits a 1 -> 1 layer of degree 8 to 100 points with Adam.  Run stage
by stage (pack, forward, loss, backward, optimizer) such a step is a dozen launches whose cost is launch and host
overhead; ``FusedTrainStep`` runs the whole step - forward, mean-squared-error loss, backward, Adam or SGD update -
as ONE kernel of one CTA (``chebykan_small_train_step``).  For models of several layers, or other losses, capture
the step in a CUDA graph instead (``kan_b200.graph.GraphedTrainStep``).
"""
from __future__ import annotations

import torch

from . import _lib, ops


def supported(batch: int, in_dim: int, out_dim: int, degree: int) -> bool:
    """True when the fused step covers this shape (at most 2048 coefficients, 16 outputs, batch * (in + out) <= 49152)."""
    return bool(_lib.load().chebykan_small_train_step_supported(batch, in_dim, out_dim, degree))


class FusedTrainStep:
    """``step = FusedTrainStep(layer, optimizer='adam', lr=0.01); loss = step(x, target)`` replaces

        optimizer.zero_grad(); loss = MSELoss()(layer(x), target); loss.backward(); optimizer.step()

    for a ``ChebyKANLayer`` in fp32.  The layer's ``cheby_coeffs`` is updated in place (its autograd version is
    bumped, so a later eager forward repacks it); ``.grad`` is not populated unless ``keep_grad=True``.  Returns the
    loss of the step's forward as a CUDA scalar (the same tensor object every call: copy it to keep a value);
    nothing synchronises.  State (Adam moments, step count) lives on
    the device, so calls can be captured in a CUDA graph as well.
    """

    def __init__(self, layer, optimizer: str = "adam", lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8,
                 keep_grad: bool = False):
        if optimizer not in ("adam", "sgd"):
            raise ValueError("optimizer must be 'adam' or 'sgd'")
        p = layer.cheby_coeffs
        if not p.is_cuda or p.dtype != torch.float32:
            raise RuntimeError("move the layer to a CUDA device first: kan_b200 has no CPU path")
        self.layer = layer
        self.optimizer = optimizer
        self.lr, self.betas, self.eps = float(lr), (float(betas[0]), float(betas[1])), float(eps)
        self.keep_grad = keep_grad
        self.exp_avg = torch.zeros_like(p.data)
        self.exp_avg_sq = torch.zeros_like(p.data)
        self.step_count = torch.zeros(1, dtype=torch.int64, device=p.device)
        self._loss = torch.empty((), dtype=torch.float32, device=p.device)
        self._fn = _lib.load().chebykan_small_train_step
        self._checked = None          # (x.data_ptr, target.data_ptr, rows) of the last validated call

    @torch.no_grad()
    def __call__(self, x: torch.Tensor, target: torch.Tensor) -> torch.Tensor:
        layer = self.layer
        p = layer.cheby_coeffs
        n_in, n_out, dp1 = p.shape
        x = x.view(-1, n_in)
        target = target.view(-1, n_out)
        B = x.shape[0]
        key = (x.data_ptr(), target.data_ptr(), B, target.shape[0])
        if key != self._checked:          # the same buffers every step (the usual loop) are validated once
            ops._require(x, "x")
            ops._require(target, "target")
            if target.shape[0] != B:
                raise RuntimeError("x and target must have the same number of rows")
            if x.device != p.device or target.device != p.device:
                raise RuntimeError("x, target and the layer must be on the same device")
            if not supported(B, n_in, n_out, dp1 - 1):
                raise RuntimeError(f"the fused step does not cover {B} x {n_in} -> {n_out}, degree {dp1 - 1}: "
                                   "use the layer with an optimizer, or kan_b200.graph.GraphedTrainStep")
            self._checked = key
        loss = self._loss
        grad = None
        if self.keep_grad:
            if p.grad is None or p.grad.shape != p.shape:
                p.grad = torch.empty_like(p.data)
            grad = p.grad
        args = (x.data_ptr(), target.data_ptr(), p.data_ptr(), self.exp_avg.data_ptr(), self.exp_avg_sq.data_ptr(),
                self.step_count.data_ptr(), loss.data_ptr(), grad.data_ptr() if grad is not None else None,
                B, n_in, n_out, dp1 - 1, 1 if self.optimizer == "adam" else 0, self.lr, self.betas[0], self.betas[1],
                self.eps, ops._stream(x))
        if torch.cuda.current_device() == p.device.index:
            rc = self._fn(*args)
        else:
            with torch.cuda.device(p.device):
                rc = self._fn(*args)
        if rc:
            _lib.check(rc, "chebykan_small_train_step")
        torch.autograd.graph.increment_version(p)      # the packed copies of the coefficients are stale now
        return loss
