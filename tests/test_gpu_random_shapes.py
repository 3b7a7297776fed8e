"""Seeded random sweep over layer shapes: every kernel (forward, dC, dx; fp32, tf32 and bf16 paths)
against the CPU oracle on shapes nobody picked by hand: ragged batches, inputs and outputs that are
not multiples of any tile, degrees from 0 to 40."""
import random

import pytest
import torch

from kan_b200 import ops
from oracle import chebykan_oracle as o
from _util import FP32_TOL, TC_TOL, assert_guards_intact, guarded, make_case

pytestmark = pytest.mark.gpu


def random_shapes(seed, n):
    rng = random.Random(seed)
    shapes = []
    for _ in range(n):
        deg = rng.choice([0, 1, 2, 3, 4, 5, 7, 8, 12, 16, 31, 32, 40])
        n_in = rng.choice([1, 2, 3, 5, 8, 13, 32, 33, 64, 65, 100, 128, 200])
        n_out = rng.choice([1, 2, 4, 7, 12, 16, 31, 32, 60, 64, 72, 128, 136, 260])
        B = rng.choice([1, 2, 31, 32, 33, 127, 128, 129, 300, 777, 1500])
        dist = rng.choice(["normal", "uniform3", "sparse"])
        shapes.append((B, n_in, n_out, deg, dist))
    return shapes


@pytest.mark.parametrize("mode,tol", [("fp32", FP32_TOL), ("tf32", TC_TOL), ("bf16", TC_TOL)])
def test_random_shape_sweep(mode, tol):
    worst = 0.0
    for k, (B, n_in, n_out, deg, dist) in enumerate(random_shapes(20240 + len(mode), 24)):
        x, coeffs, dy = make_case(B, n_in, n_out, deg, dist, seed=1000 + k)
        c_fwd = coeffs.bfloat16().float() if mode == "bf16" else coeffs
        y_ref = o.forward(x, c_fwd)
        _, dC_ref, dx_ref = o.forward_backward(x, coeffs, dy)
        xd, cd, dyd = x.cuda(), coeffs.cuda(), dy.cuda()
        y, yw = guarded((B, n_out))
        ops.forward(xd, ops.pack_coeffs(cd, mode), n_in, n_out, deg, mode, out=y)
        dC, dCw = guarded((n_in, n_out, deg + 1))
        ops.bwd_dcoeff(xd, dyd, n_in, n_out, deg, mode, out=dC)
        dx, dxw = guarded((B, n_in))
        ops.bwd_dx(xd, dyd, cd, mode, out=dx)
        torch.cuda.synchronize()
        ops.check_status()
        for v, w in ((y, yw), (dC, dCw), (dx, dxw)):
            assert_guards_intact(v, w)
        # tiny shapes have no averaging: one bf16 product carries up to 2^-8 relative error on its own
        lim = tol if (mode == "fp32" or n_in * (deg + 1) >= 64) else 3 * tol
        errs = (o.rel_l2(y.cpu(), y_ref), o.rel_l2(dC.cpu(), dC_ref), o.rel_l2(dx.cpu(), dx_ref))
        assert max(errs) <= lim, ((B, n_in, n_out, deg, dist), mode, errs)
        worst = max(worst, *errs)
    assert worst > 0.0
