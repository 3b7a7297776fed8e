"""CUDA-graph capture of a whole training step for launch-bound models.

Small ChebyKAN models (a 1 -> 1 layer on 100 points, a 784 -> 64 -> 10
classifier on 256 samples) spend their step in launch overhead: a dozen
kernels of a few microseconds each.  ``GraphedTrainStep`` records forward,
loss, backward and optimizer update of a single-GPU model once and replays
them as one graph launch.  Inputs and targets are static device buffers that
the caller overwrites in place between replays.
"""
from __future__ import annotations

from typing import Callable

import torch

from . import dp, ops

# warm-up runs on a side stream while older AccumulateGrad nodes belong to the default stream; the
# mismatch is intended here and harmless (the streams are joined before and after)
torch.autograd.graph.set_warn_on_accumulate_grad_stream_mismatch(False)


class GraphedTrainStep:
    def __init__(self, model: torch.nn.Module, loss_fn: Callable, optimizer, x: torch.Tensor, target: torch.Tensor,
                 warmup: int = 3, status_every: int = 256):
        """`optimizer` must be graph-capturable (kan_b200.optim.SGD, or Adam(capturable=True))."""
        self.status_every = int(status_every)
        self._replays = 0
        if getattr(optimizer, "capturable", True) is False:
            raise ValueError("use kan_b200.optim.Adam(..., capturable=True) for a graphed step")
        self.model, self.loss_fn, self.opt = model, loss_fn, optimizer
        self.x, self.target = x, target
        self.grads = dp.FlatGradBuffer(model.parameters())
        self.loss = None
        side = torch.cuda.Stream(device=x.device)
        side.wait_stream(torch.cuda.current_stream(x.device))
        with torch.cuda.stream(side):
            for _ in range(warmup):          # also builds every lazily created kernel attribute / buffer
                self._eager_step()
        torch.cuda.current_stream(x.device).wait_stream(side)
        torch.cuda.synchronize(x.device)
        ops.check_status()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self._eager_step()

    def _eager_step(self):
        self.grads.zero()
        self.loss = self.loss_fn(self.model(self.x), self.target)
        self.loss.backward()
        self.opt.step()

    def __call__(self) -> torch.Tensor:
        """Replay one step; returns the (device) loss tensor of that step.

        The replayed kernels write the parameters through raw pointers, so every
        replay bumps each parameter's autograd version: anything keyed on it (the
        layers' packed-coefficient caches, which an eager forward between replays
        consults) sees that the coefficients changed.  Every `status_every`
        replays (default 256; 0 = never) the device status word of the bounded
        waits is read back, which synchronises: a kernel that gave up a wait
        raises here instead of training on unwritten buffers."""
        self.graph.replay()
        for p in self.grads.params:
            torch.autograd.graph.increment_version(p)
        self._replays += 1
        if self.status_every and self._replays % self.status_every == 0:
            ops.check_status(self.x.device)
        return self.loss
