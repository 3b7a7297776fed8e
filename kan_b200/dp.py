"""Batch-sharded data parallelism for ChebyKAN models on one multi-GPU host.

Rows of the batch are independent (the reference flattens every leading
dimension into rows, kan/layers/chebykan.py:64), so inference needs no
communication: each rank runs the layer on its block of rows with replicated
coefficients.  Training adds exactly one exchange per step: a sum all-reduce
of the coefficient gradients, issued on ONE flat buffer that every
parameter's ``.grad`` aliases, through ``torch.distributed`` (NCCL over
NVLink on GPUs; gloo in the CPU tests of this host logic).
"""
from __future__ import annotations

import os
from typing import Iterable, List, Tuple

import torch
import torch.distributed as dist


def shard_rows(n_rows: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous block [begin, end) of rows owned by `rank`; sizes differ by at most one."""
    base, rem = divmod(n_rows, world)
    begin = rank * base + min(rank, rem)
    return begin, begin + base + (1 if rank < rem else 0)


class FlatGradBuffer:
    """One flat fp32 buffer holding every parameter's gradient.

    After construction ``p.grad`` is a view into the buffer for every
    parameter, so backward kernels write their results straight into it and
    one collective covers all layers.
    """

    def __init__(self, params: Iterable[torch.nn.Parameter]):
        self.params: List[torch.nn.Parameter] = [p for p in params if p.requires_grad]
        if not self.params:
            raise ValueError("no trainable parameters")
        dev = self.params[0].device
        sizes = [(p.numel() + 3) // 4 * 4 for p in self.params]   # keep every view 16-byte aligned
        self.flat = torch.zeros(sum(sizes), dtype=torch.float32, device=dev)
        self._views: List[torch.Tensor] = []
        off = 0
        for p, n in zip(self.params, sizes):
            self._views.append(self.flat[off:off + p.numel()].view_as(p))
            off += n
        self.attach()

    def attach(self) -> None:
        """Make every ``p.grad`` the parameter's view of the flat buffer again.

        ``optimizer.zero_grad()`` with ``set_to_none=True`` (torch's default) drops ``p.grad``; the next backward
        then installs a fresh tensor that the collective would not see.  A gradient found detached is copied into
        its view (so nothing a backward already produced is lost) and re-attached."""
        for p, v in zip(self.params, self._views):
            g = p.grad
            if g is None:
                v.zero_()
                p.grad = v
            elif g.data_ptr() != v.data_ptr():
                v.copy_(g)
                p.grad = v

    def zero(self) -> None:
        """Clear every gradient (use this, or ``zero_grad(set_to_none=False)``, instead of dropping ``p.grad``)."""
        self.flat.zero_()
        self.attach()

    def all_reduce(self, group=None, async_op: bool = False):
        """Sum the gradients over the ranks of `group` (no-op for a single process)."""
        self.attach()
        if not dist.is_available() or not dist.is_initialized() or dist.get_world_size(group) == 1:
            return None
        if self.flat.is_cuda and os.environ.get("KAN_B200_NVTX", "0") == "1":
            with torch.cuda.nvtx.range("chebykan.allreduce_dC"):
                return dist.all_reduce(self.flat, op=dist.ReduceOp.SUM, group=group, async_op=async_op)
        return dist.all_reduce(self.flat, op=dist.ReduceOp.SUM, group=group, async_op=async_op)


def world_info() -> Tuple[int, int]:
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank(), dist.get_world_size()
    return 0, 1
