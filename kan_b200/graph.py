"""CUDA-graph capture of a whole training step for launch-bound models.

Small ChebyKAN models (a 1 -> 1 layer on 100 points, a 784 -> 64 -> 10
classifier on 256 samples) spend their step in launch overhead: a dozen
kernels of a few microseconds each.  ``GraphedTrainStep`` records forward,
loss, backward and optimizer update of a model once and replays them as one
graph launch.  Inputs and targets are static device buffers that the caller
overwrites in place between replays.

Data-parallel training is launch-bound sooner: sharding a batch over N GPUs
divides the kernels' time by N but not the host's time to issue them (about
0.5 ms for a two-layer model), so from a few hundred thousand rows per GPU
down the step waits for the host.  With ``torch.distributed`` initialised
(NCCL) the recorded step includes the all-reduce of the flat gradient buffer,
so every rank replays forward, backward, collective and update as one launch.
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
                 warmup: int = 3, status_every: int = 256, all_reduce_grads: bool = True, group=None):
        """`optimizer` must be graph-capturable (kan_b200.optim.SGD, or Adam(capturable=True)).

        With more than one rank in `group` (default: the world) and `all_reduce_grads`, the gradients are summed
        over the ranks between backward and the update, inside the graph; the loss function then has to
        normalise by the GLOBAL batch (e.g. ``mse_loss(..., n_mean=global_rows * out)``).  The warm-up steps run
        the collective eagerly first, so the communicator exists before the capture starts."""
        self.status_every = int(status_every)
        self.group = group
        self._reduce = bool(all_reduce_grads) and dp.world_info_of(group)[1] > 1
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
        if self._reduce:
            self.grads.all_reduce(self.group)
        self.opt.step()

    def close(self) -> None:
        """Destroy the recorded graph (replaying afterwards raises).  A graph that holds a captured collective keeps
        the NCCL communicator busy: ``torch.distributed.destroy_process_group`` blocks until the graph is gone,
        so a data-parallel job calls this (or drops the object) before it shuts the process group down."""
        if getattr(self, "graph", None) is not None:
            torch.cuda.synchronize(self.x.device)
            self.graph.reset()
            self.graph = None

    def __del__(self):
        try:
            self.close()
        except Exception:        # interpreter shutdown: the CUDA context may be gone already
            pass

    def __call__(self) -> torch.Tensor:
        """Replay one step; returns the (device) loss tensor of that step.

        The replayed kernels write the parameters through raw pointers, so every
        replay bumps each parameter's autograd version: anything keyed on it (the
        layers' packed-coefficient caches, which an eager forward between replays
        consults) sees that the coefficients changed.  Every `status_every`
        replays (default 256; 0 = never) the device status word of the bounded
        waits is read back, which synchronises: a kernel that gave up a wait
        raises here instead of training on unwritten buffers."""
        if self.graph is None:
            raise RuntimeError("this graphed step was closed")
        self.graph.replay()
        for p in self.grads.params:
            torch.autograd.graph.increment_version(p)
        self._replays += 1
        if self.status_every and self._replays % self.status_every == 0:
            ops.check_status(self.x.device)
        return self.loss
