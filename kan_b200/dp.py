"""Batch-sharded data parallelism for ChebyKAN models on one multi-GPU host.

Rows of the batch are independent (the reference flattens every leading
dimension into rows, kan/layers/chebykan.py:64), so inference needs no
communication: each rank runs the layer on its block of rows with replicated
coefficients.  Training adds exactly one exchange per step: a sum all-reduce
of the coefficient gradients, issued on ONE flat buffer that every
parameter's ``.grad`` aliases, through ``torch.distributed`` (NCCL over
NVLink on GPUs; gloo in the CPU tests of this host logic).

A second sharding axis, for a layer whose coefficients should not be
replicated: the OUTPUT dimension.  ``coefficients[in, out, deg+1]`` splits
along ``out`` into independent layers (each output is its own sum over inputs
and degrees, the einsum 'bid,iod->bo' of kan/basis/chebyshev.py:101), so rank r
holds ``coefficients[:, o_r : o_{r+1}, :]``, computes its columns of y from the
full input, and the only exchanges are a sum all-reduce of dx in backward and -
when the next consumer needs whole rows - an all-gather of y
(``OutputParallel``).
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


def world_info_of(group=None) -> Tuple[int, int]:
    """(rank, size) within `group` (the world when None); (0, 1) without an initialised process group."""
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank(group), dist.get_world_size(group)
    return 0, 1


# ---------------------------------------------------------------------------------------------------------------
# sharding over the output dimension
# ---------------------------------------------------------------------------------------------------------------
def shard_outputs(n_out: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous block [begin, end) of output columns owned by `rank` (same rule as ``shard_rows``)."""
    return shard_rows(n_out, rank, world)


class _SumGradAcrossRanks(torch.autograd.Function):
    """Identity in forward; in backward the incoming gradient is summed over the ranks of the group: every rank
    computes the part of dx that flows through its own output columns."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x.view_as(x)

    @staticmethod
    def backward(ctx, dx):
        dx = dx.contiguous()
        dist.all_reduce(dx, op=dist.ReduceOp.SUM, group=ctx.group)
        return dx, None


class _GatherColumns(torch.autograd.Function):
    """All-gather of the ranks' column blocks into whole rows; backward keeps this rank's columns of the gradient."""

    @staticmethod
    def forward(ctx, y_local, sizes, rank, group):
        ctx.sizes, ctx.rank = sizes, rank
        # equal shapes on every rank: blocks are padded to the widest shard (shards differ by at most one column)
        width = max(sizes)
        padded = y_local.new_zeros(y_local.shape[0], width)
        padded[:, :y_local.shape[1]] = y_local
        bufs = [torch.empty_like(padded) for _ in sizes]
        dist.all_gather(bufs, padded, group=group)
        return torch.cat([b[:, :n] for b, n in zip(bufs, sizes)], dim=1)

    @staticmethod
    def backward(ctx, dy):
        begin = sum(ctx.sizes[:ctx.rank])
        return dy[:, begin:begin + ctx.sizes[ctx.rank]].contiguous(), None, None, None


class OutputParallel(torch.nn.Module):
    """A KAN layer sharded over its output dimension.

    ``make_layer(out_local)`` builds this rank's shard (any layer class of this package with ``out_local`` outputs);
    ``full_coefficients`` ([in, out, deg+1], identical on every rank, e.g. from a checkpoint) is optional and is
    sliced into the shard's parameter.  ``forward(x)`` takes the full input rows on every rank and returns this
    rank's columns of y, or whole rows with ``gather_output=True``.  Without an initialised process group (or with
    one rank) it is the plain layer.
    """

    def __init__(self, make_layer, n_out: int, full_coefficients: torch.Tensor | None = None,
                 gather_output: bool = False, group=None):
        super().__init__()
        self.group = group
        self.gather_output = gather_output
        self.rank, self.world = 0, 1
        if dist.is_available() and dist.is_initialized():
            self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.n_out = n_out
        self.sizes = [shard_outputs(n_out, r, self.world)[1] - shard_outputs(n_out, r, self.world)[0]
                      for r in range(self.world)]
        if min(self.sizes) < 1:
            raise ValueError(f"{n_out} outputs cannot be split over {self.world} ranks")
        self.begin, self.end = shard_outputs(n_out, self.rank, self.world)
        self.shard = make_layer(self.end - self.begin)
        if full_coefficients is not None:
            with torch.no_grad():
                self.shard.get_coefficients().copy_(full_coefficients[:, self.begin:self.end, :])

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.world == 1:
            return self.shard(x)
        y = self.shard(_SumGradAcrossRanks.apply(x, self.group))
        if self.gather_output:
            y = _GatherColumns.apply(y, self.sizes, self.rank, self.group)
        return y

    def full_coefficients(self) -> torch.Tensor:
        """The whole [in, out, deg+1] tensor, gathered from the shards (for a checkpoint)."""
        c = self.shard.get_coefficients().detach()
        if self.world == 1:
            return c.clone()
        width = max(self.sizes)                      # equal shapes on every rank, as in _GatherColumns
        padded = torch.zeros(c.shape[0], width, c.shape[2], dtype=c.dtype, device=c.device)
        padded[:, :c.shape[1]] = c
        bufs = [torch.empty_like(padded) for _ in range(self.world)]
        dist.all_gather(bufs, padded, group=self.group)
        return torch.cat([b[:, :n] for b, n in zip(bufs, self.sizes)], dim=1)
