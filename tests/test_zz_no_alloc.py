"""GPU test of chebykan_bwd_dcoeff_static, the coefficient-gradient entry point
for callers that cannot allocate device memory (they only receive raw pointers
from a host that owns the whole GPU, or run where CUDA allocation calls are
forbidden).  It must give what chebykan_bwd_dcoeff gives with a caller-made
workspace, call after call, although all calls share one built-in scratch array
that still holds whatever the previous call left there.

Collected last on purpose: a run that stops at the first failure has then
already run every other test.  It also passes alone in a fresh process."""
import pytest
import torch

from kan_b200 import _lib, ops
from oracle import chebykan_oracle as o
from _util import FP32_TOL, make_case

pytestmark = pytest.mark.gpu


def static_dcoeff(x, dy, n_in, n_out, deg, accumulate=False, out=None):
    lib = _lib.load()
    if out is None:
        out = torch.full((n_in, n_out, deg + 1), float("nan"), device="cuda")
    rc = lib.chebykan_bwd_dcoeff_static(x.data_ptr(), dy.data_ptr(), out.data_ptr(), x.shape[0], n_in, n_out,
                                        deg, int(accumulate), torch.cuda.current_stream().cuda_stream)
    return rc, out


def test_static_scratch_variant_matches_workspace_variant_twice_in_a_row():
    lib = _lib.load()
    # two different shapes back to back, both large enough to split the batch and use scratch;
    # the second call finds the first call's partial sums still in the array
    shapes = [(20000, 8, 8, 4), (65536, 64, 64, 8)]
    for B, n_in, n_out, deg in shapes:
        assert lib.chebykan_workspace_bytes(_lib.OP_BWD_DCOEFF, B, n_in, n_out, deg, 0) > 0
        x, coeffs, dy = make_case(B, n_in, n_out, deg, seed=B % 97)
        xd, dyd = x.cuda(), dy.cuda()
        expect = ops.bwd_dcoeff(xd, dyd, n_in, n_out, deg, "fp32")
        for _ in range(2):
            rc, got = static_dcoeff(xd, dyd, n_in, n_out, deg)
            assert rc == 0, _lib.strerror(rc)
            torch.cuda.synchronize()
            assert o.rel_l2(got.cpu(), expect.cpu()) <= FP32_TOL
        _, dC_ref, _ = o.forward_backward(x[:4096], coeffs, dy[:4096], need_dx=False)
        rc, part = static_dcoeff(xd[:4096].contiguous(), dyd[:4096].contiguous(), n_in, n_out, deg)
        assert rc == 0 and o.rel_l2(part.cpu(), dC_ref) <= FP32_TOL
    # accumulate adds onto what the caller's buffer holds
    B, n_in, n_out, deg = shapes[0]
    x, _, dy = make_case(B, n_in, n_out, deg, seed=B % 97)
    xd, dyd = x.cuda(), dy.cuda()
    expect = ops.bwd_dcoeff(xd, dyd, n_in, n_out, deg, "fp32")
    acc = torch.zeros(n_in, n_out, deg + 1, device="cuda")
    for _ in range(2):
        rc, _ = static_dcoeff(xd, dyd, n_in, n_out, deg, accumulate=True, out=acc)
        assert rc == 0
    assert o.rel_l2(acc.cpu(), 2 * expect.cpu()) <= FP32_TOL


def test_static_scratch_variant_refuses_what_does_not_fit():
    lib = _lib.load()
    B, n_in, n_out, deg = 80000, 16, 128, 7
    assert lib.chebykan_workspace_bytes(_lib.OP_BWD_DCOEFF, B, n_in, n_out, deg, 0) > (16 << 20)
    x = torch.zeros(B, n_in, device="cuda")
    dy = torch.zeros(B, n_out, device="cuda")
    rc, _ = static_dcoeff(x, dy, n_in, n_out, deg)
    assert rc == -8 and "16 MiB" in _lib.strerror(rc)
    torch.cuda.synchronize()
