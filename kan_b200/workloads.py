"""Seeded synthetic inputs and model shapes of the five benchmark configurations.

No dataset is read: every tensor is generated on the CPU from a seeded
``torch.Generator`` with the shapes, sizes and value distributions the
configurations name.  Configuration 2's input only imitates the sparsity of an
image-like tensor (about 80 % exact zeros); it contains no dataset items.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Callable, List, Tuple

import torch
import torch.nn as nn


@dataclass(frozen=True)
class Config:
    name: str
    batch: int
    layers: Tuple[Tuple[int, int, int], ...]   # (in, out, degree) per ChebyKAN layer
    layernorm_between: bool
    task: str                                  # 'fwd' | 'train'
    loss: str = ''                             # 'mse' | 'ce'
    optimizer: str = ''                        # 'adam' | 'sgd'
    lr: float = 0.0
    seed: int = 0


CONFIGS = {
    'cfg1': Config('cfg1', 100, ((1, 1, 8),), False, 'train', 'mse', 'adam', 0.01, 1001),
    'cfg2': Config('cfg2', 256, ((784, 64, 4), (64, 10, 4)), True, 'train', 'ce', 'adam', 1e-3, 1002),
    'cfg3': Config('cfg3', 65536, ((1024, 1024, 8),), False, 'fwd', seed=1003),
    'cfg4': Config('cfg4', 32768, ((2048, 2048, 4),) * 4, True, 'fwd', seed=1004),
    'cfg5': Config('cfg5', 1048576, ((64, 64, 32), (64, 64, 32)), False, 'train', 'mse', 'sgd', 1e-2, 1005),
}


def flops_per_sample(cfg: Config) -> int:
    """Forward FLOPs per sample: 2 * in * (deg+1) * out summed over the layers."""
    return sum(2 * i * (d + 1) * o for i, o, d in cfg.layers)


def make_inputs(cfg: Config, batch: int | None = None, seed: int | None = None):
    """(x, target) on the CPU for `batch` rows (default: the configuration's batch)."""
    B = cfg.batch if batch is None else batch
    g = torch.Generator().manual_seed(cfg.seed if seed is None else seed)
    n_in = cfg.layers[0][0]
    n_out = cfg.layers[-1][1]
    if cfg.name == 'cfg1':
        # 100 points linspace(-1, 1) shaped [B, 1]; target sin(2 pi x)
        x = torch.linspace(-1.0, 1.0, B, dtype=torch.float64).to(torch.float32).view(B, 1)
        return x, torch.sin(2 * math.pi * x)
    if cfg.name == 'cfg2':
        x = torch.rand(B, n_in, generator=g)
        x = torch.where(torch.rand(B, n_in, generator=g) < 0.8, torch.zeros(()), x)
        labels = torch.randint(0, n_out, (B,), generator=g)
        return x, labels
    if cfg.name in ('cfg3', 'cfg4'):
        return torch.randn(B, n_in, generator=g), None
    if cfg.name == 'cfg5':
        x = torch.rand(B, n_in, generator=g) * 6.0 - 3.0
        target = torch.sin(x).sum(1, keepdim=True).expand(-1, n_out).contiguous()
        return x, target
    raise KeyError(cfg.name)


def build_model(cfg: Config, layer_cls: Callable[..., nn.Module], seed: int | None = None, **layer_kw) -> nn.Sequential:
    """Sequential stack of the configuration, built on the CPU under a fixed seed.

    Given the same seed, the reference's layer class and this package's layer
    class draw identical coefficients (both consume the global CPU RNG the same
    way), so the two models start from the same weights.
    """
    torch.manual_seed(cfg.seed if seed is None else seed)
    mods: List[nn.Module] = []
    for k, (i, o, d) in enumerate(cfg.layers):
        if k > 0 and cfg.layernorm_between:
            mods.append(nn.LayerNorm(i))
        mods.append(layer_cls(i, o, d, **layer_kw))
    return nn.Sequential(*mods)


def loss_fn(cfg: Config):
    if cfg.loss == 'mse':
        return nn.MSELoss()
    if cfg.loss == 'ce':
        return nn.CrossEntropyLoss()
    raise KeyError(cfg.loss)
