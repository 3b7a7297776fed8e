"""SGD and Adam whose updates run in the library's CUDA kernels.

Stand in for ``torch.optim.SGD(params, lr)`` and ``torch.optim.Adam(params,
lr)`` as the reference's training loop uses them (README.md:59-66): no
momentum / weight decay for SGD; Adam with betas (0.9, 0.999), eps 1e-8, bias
correction, no weight decay, no amsgrad.  Works on any contiguous fp32 CUDA
parameter (ChebyKAN coefficients, LayerNorm weights, ...).  ``grad_scale``
multiplies every gradient first (1/world_size after a sum all-reduce).
"""
from __future__ import annotations

import torch

from . import ops


def _bump(p: torch.Tensor) -> None:
    # the kernels write through the raw pointer; tell autograd the tensor changed
    torch.autograd.graph.increment_version(p)


class _Base:
    def __init__(self, params, lr: float):
        self.params = [p for p in params]
        if not self.params:
            raise ValueError("optimizer got an empty parameter list")
        for p in self.params:
            if not p.is_cuda or p.dtype != torch.float32 or not p.is_contiguous():
                raise RuntimeError("kan_b200 optimizers need contiguous fp32 CUDA parameters")
        self.lr = float(lr)
        self.grad_scale = 1.0
        # opt-in: read the kernels' status word every `check_status_every` steps (a device synchronisation) and
        # raise if a bounded wait gave up since the last check; 0 = never
        self.check_status_every = 0
        self._steps = 0

    def _after_step(self) -> None:
        self._steps += 1
        if self.check_status_every and self._steps % self.check_status_every == 0:
            ops.check_status(self.params[0].device)

    def zero_grad(self, set_to_none: bool = False) -> None:
        """Zero the gradients in place by default (torch's optimizers drop them): a gradient that aliases a
        ``dp.FlatGradBuffer`` stays attached to it."""
        for p in self.params:
            if p.grad is not None:
                if set_to_none:
                    p.grad = None
                else:
                    p.grad.zero_()


class SGD(_Base):
    def __init__(self, params, lr: float = 1e-3):
        super().__init__(params, lr)

    @torch.no_grad()
    def step(self) -> None:
        for p in self.params:
            if p.grad is None:
                continue
            ops.sgd_step(p.data, p.grad.contiguous(), self.lr, self.grad_scale)
            _bump(p)
        self._after_step()


class Adam(_Base):
    """``capturable=True`` keeps the step counters in device memory so that ``step()`` can be
    captured in a CUDA graph and replayed (the host-side counter of the default mode would be
    frozen into the graph)."""

    def __init__(self, params, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8, capturable: bool = False):
        super().__init__(params, lr)
        self.betas = (float(betas[0]), float(betas[1]))
        self.eps = float(eps)
        self.capturable = bool(capturable)
        self.state = {}
        if self.capturable:
            for p in self.params:     # allocate before any capture
                self._state(p)

    def _state(self, p):
        st = self.state.get(p)
        if st is None:
            st = {"step": 0, "exp_avg": torch.zeros_like(p), "exp_avg_sq": torch.zeros_like(p)}
            if self.capturable:
                st["step_dev"] = torch.zeros(1, dtype=torch.int64, device=p.device)
            self.state[p] = st
        return st

    @torch.no_grad()
    def step(self) -> None:
        for p in self.params:
            if p.grad is None:
                continue
            st = self._state(p)
            if self.capturable:
                ops.adam_step_graph(p.data, p.grad.contiguous(), st["exp_avg"], st["exp_avg_sq"], st["step_dev"],
                                    self.lr, self.betas[0], self.betas[1], self.eps, self.grad_scale)
            else:
                st["step"] += 1
                ops.adam_step(p.data, p.grad.contiguous(), st["exp_avg"], st["exp_avg_sq"], st["step"], self.lr,
                              self.betas[0], self.betas[1], self.eps, self.grad_scale)
            _bump(p)
        self._after_step()
