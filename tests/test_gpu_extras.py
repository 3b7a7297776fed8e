"""GPU tests of what sits either side of the layer kernels: the fused MSE loss, the basis object's own
methods, the graphed training step's interaction with the eager path, and short training trajectories
of the basis-bound configuration against the oracle model."""
import pytest
import torch

import kan_b200
from kan_b200 import ops, workloads
from oracle import chebykan_oracle as o
from _util import FP32_TOL, TC_TOL, OracleLayer

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("shape", [(1000, 64), (333, 7), (1, 1), (4099, 3)])
def test_mse_loss_matches_torch(shape):
    g = torch.Generator().manual_seed(sum(shape))
    y = torch.randn(*shape, generator=g)
    t = torch.randn(*shape, generator=g)
    yr = y.clone().requires_grad_(True)
    loss_ref = torch.nn.functional.mse_loss(yr, t)
    (loss_ref * 3.0).backward()
    yd = y.cuda().requires_grad_(True)
    loss = kan_b200.mse_loss(yd, t.cuda())
    (loss * 3.0).backward()                        # a chain-rule factor other than 1 reaches the stored gradient
    assert abs(float(loss) - float(loss_ref)) <= 1e-6 * abs(float(loss_ref))
    assert o.rel_l2(yd.grad.cpu(), yr.grad) <= 1e-6
    # plain backward (factor exactly 1) and bitwise repeatability of the fixed-order reduction
    yd2 = y.cuda().requires_grad_(True)
    l2 = kan_b200.MSELoss()(yd2, t.cuda())
    l2.backward()
    assert o.rel_l2(yd2.grad.cpu(), yr.grad / 3.0) <= 1e-6
    l3, _ = ops.mse_loss_grad(y.cuda(), t.cuda())
    assert torch.equal(l2.detach(), l3)
    # a global divisor (sharded batch): loss and gradient scale by n / n_mean
    l4, dy4 = ops.mse_loss_grad(y.cuda(), t.cuda(), n_mean=4 * y.numel())
    assert abs(float(l4) - float(loss_ref) / 4) <= 1e-6 * abs(float(loss_ref))
    assert o.rel_l2(dy4.cpu(), yr.grad / 12.0) <= 1e-6


def test_basis_object_surface():
    basis = kan_b200.ChebyshevBasis(8)
    x = torch.randn(37, 5)
    t = basis.normalize_input(x.cuda())
    assert o.rel_l2(t.cpu(), torch.tanh(x)) <= 1e-7
    phi = basis.basis_functions(t)
    assert phi.shape == (37, 5, 9)
    assert o.rel_l2(phi.cpu(), o.basis_closed_form(torch.tanh(x), 8)) <= FP32_TOL
    # out-of-domain points are clamped like the reference's closed form (acos of a clamped value)
    edge = basis.basis_functions(torch.tensor([[1.5, -2.0]], device="cuda")).cpu()
    assert torch.equal(edge[0, 0], torch.ones(9)) and torch.equal(edge[0, 1], torch.tensor([1., -1.] * 4 + [1.]))
    coeffs = torch.randn(5, 3, 9) * 0.2
    d0 = basis.derivative(x.cuda(), coeffs.cuda(), order=0)
    assert o.rel_l2(d0.cpu(), o.forward(x, coeffs)) <= FP32_TOL
    xr = x.clone().requires_grad_(True)
    y = o.forward(xr, coeffs)
    ref = torch.stack([torch.autograd.grad(y[:, k].sum(), xr, retain_graph=True)[0].sum(-1) for k in range(3)], 1)
    assert o.rel_l2(basis.derivative(x.cuda(), coeffs.cuda()).cpu(), ref) <= FP32_TOL
    with pytest.raises(NotImplementedError):
        basis.derivative(x.cuda(), coeffs.cuda(), order=2)


@pytest.mark.parametrize("mode", ["fp32", "tf32"])
def test_eager_forward_between_graph_replays_sees_current_coefficients(mode):
    """Replays update the coefficients through raw pointers; an eager forward in between must not reuse a packed
    copy of older coefficients."""
    torch.manual_seed(4)
    layer = kan_b200.ChebyKANLayer(48, 40, 5, math_mode=mode).cuda()
    x = torch.randn(256, 48, device="cuda")
    tgt = torch.randn(256, 40, device="cuda")
    opt = kan_b200.optim.SGD(layer.parameters(), lr=0.5)
    step = kan_b200.graph.GraphedTrainStep(layer, torch.nn.functional.mse_loss, opt, x, tgt)
    tol = FP32_TOL if mode == "fp32" else TC_TOL
    for _ in range(3):
        for _ in range(4):
            step()
        with torch.no_grad():
            y = layer(x)                       # eager: goes through the layer's packed-coefficient cache
        fresh = ops.forward(x, ops.pack_coeffs(layer.cheby_coeffs.detach(), mode), 48, 40, 5, mode)
        assert torch.equal(y, fresh)
        assert o.rel_l2(y.cpu(), o.forward(x.cpu(), layer.cheby_coeffs.detach().cpu())) <= tol


@pytest.mark.parametrize("mode,tol", [("fp32", 2e-5), ("fp32x3", 2e-5), ("tf32", TC_TOL), ("bf16", TC_TOL)])
def test_cfg5_training_trajectory_vs_oracle_model(mode, tol):
    """Configuration 5 (64 -> 64 -> 64, degree 32, x ~ U(-3,3), MSE, SGD 1e-2) at a reduced batch: three full steps of
    the model (forward, fused loss, backward, optimizer) against the oracle model under torch's MSE and SGD.  The
    coefficients move by about 10 % over these steps and the gradient doubles from step to step, so a kernel's error in
    one step is amplified in the next: the end point is held to 2.5 x the per-kernel tolerance."""
    cfg = workloads.CONFIGS["cfg5"]
    B = 4096
    x, tgt = workloads.make_inputs(cfg, batch=B)
    ref = workloads.build_model(cfg, OracleLayer)
    ours = workloads.build_model(cfg, kan_b200.ChebyKANLayer, math_mode=mode).cuda()
    opt_ref = torch.optim.SGD(ref.parameters(), lr=cfg.lr)
    opt = kan_b200.optim.SGD(list(ours.parameters()), lr=cfg.lr)
    xd, td = x.cuda(), tgt.cuda()
    start = [p.detach().clone() for p in ref.parameters()]
    for step in range(3):
        opt_ref.zero_grad()
        loss_ref = torch.nn.functional.mse_loss(ref(x), tgt)
        loss_ref.backward()
        opt_ref.step()
        opt.zero_grad()
        loss = kan_b200.mse_loss(ours(xd), td)
        loss.backward()
        opt.step()
        assert abs(float(loss.detach()) - float(loss_ref.detach())) <= tol * abs(float(loss_ref.detach())), step
    ops.check_status()
    for p0, a, b in zip(start, ref.parameters(), ours.parameters()):
        assert o.rel_l2(a.detach(), p0) > 1e-2                 # the steps did change the coefficients
        assert o.rel_l2(b.detach().cpu(), a.detach()) <= 2.5 * tol
        assert o.rel_l2(b.detach().cpu() - p0, a.detach() - p0) <= 25 * tol      # the update itself, not just the end point


# ---------------------------------------------------------------------------------------------------------------
# Full BASELINE sizes, through properties that need no CPU oracle run of that size: rows are independent, so a
# sample of rows of the full-size result can be checked against the oracle; the coefficient gradient is additive
# over row blocks and linear in dY.
# ---------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("mode,tol", [("bf16", TC_TOL), ("tf32", TC_TOL)])
def test_full_size_cfg4_stack_row_sample(mode, tol):
    """Configuration 4 at full size (32768 rows through 4 x (2048 -> 2048, degree 4) with LayerNorms): 48 sampled rows of
    the GPU result against the oracle model, for the plain and the LayerNorm-fused stack."""
    cfg = workloads.CONFIGS["cfg4"]
    ref = workloads.build_model(cfg, OracleLayer)
    ours = workloads.build_model(cfg, kan_b200.ChebyKANLayer, math_mode=mode)
    if mode == "bf16":            # coefficients stored in bf16: the oracle evaluates with the same rounded values
        with torch.no_grad():
            for m in ref:
                if hasattr(m, "cheby_coeffs"):
                    m.cheby_coeffs.copy_(m.cheby_coeffs.bfloat16().float())
    ours = ours.cuda()
    x, _ = workloads.make_inputs(cfg)
    xd = x.cuda()
    rows = torch.cat([torch.tensor([0, 1, 127, 128, 255, 256, 16383, 16384, 32767]), torch.arange(20000, 20039)])
    with torch.no_grad():
        y = ours(xd)
        y_fused = kan_b200.fuse_layernorm(ours)(xd)
        y_ref = ref(x[rows])
    ops.check_status()
    assert y.shape == (cfg.batch, 2048)
    # rounding accumulates over the four layers (each LayerNorm rescales the previous layer's error with its signal):
    # the same bound as the reduced-size stack tests, 1.5 x the single-kernel tolerance per layer
    err, err_fused = o.rel_l2(y[rows.cuda()].cpu(), y_ref), o.rel_l2(y_fused[rows.cuda()].cpu(), y_ref)
    print(f"cfg4 full size, {mode}: rel-L2 {err:.3e} (plain), {err_fused:.3e} (LayerNorm fused)")
    assert err <= 1.5 * tol * 4
    assert err_fused <= 1.1 * err + 1e-4


@pytest.mark.parametrize("mode", ["tf32", "bf16"])
def test_full_size_cfg5_layer_properties(mode):
    """Configuration 5's layer at full size (1048576 x 64 -> 64, degree 32, x ~ U(-3,3)): forward and dx on sampled rows
    against the oracle; dC additive over the two halves of the batch, linear in dY, and equal to the oracle on a
    32768-row block."""
    B, n_in, n_out, deg = 1048576, 64, 64, 32
    g = torch.Generator(device="cuda").manual_seed(5)
    x = torch.rand(B, n_in, device="cuda", generator=g) * 6 - 3
    dy = torch.randn(B, n_out, device="cuda", generator=g)
    coeffs = torch.randn(n_in, n_out, deg + 1, device="cuda", generator=g) / (n_in * (deg + 1))
    packed = ops.pack_coeffs(coeffs, mode)
    y = ops.forward(x, packed, n_in, n_out, deg, mode)
    dx = ops.bwd_dx(x, dy, coeffs, mode)
    dC = ops.bwd_dcoeff(x, dy, n_in, n_out, deg, mode)
    torch.cuda.synchronize()
    ops.check_status()
    rows = torch.cat([torch.tensor([0, 1, 127, 128, 255, 256, 524287, 524288, B - 1]), torch.arange(700000, 700055)]).cuda()
    c_cpu = coeffs.cpu()
    c_fwd = c_cpu.bfloat16().float() if mode == "bf16" else c_cpu
    y_ref = o.forward(x[rows].cpu(), c_fwd)
    _, _, dx_ref = o.forward_backward(x[rows].cpu(), c_cpu, dy[rows].cpu())
    assert o.rel_l2(y[rows].cpu(), y_ref) <= TC_TOL
    assert o.rel_l2(dx[rows].cpu(), dx_ref) <= TC_TOL
    # additivity over row blocks (each half is its own launch with its own batch split and dY scale)
    h = B // 2
    dC_a = ops.bwd_dcoeff(x[:h].contiguous(), dy[:h].contiguous(), n_in, n_out, deg, mode)
    dC_b = ops.bwd_dcoeff(x[h:].contiguous(), dy[h:].contiguous(), n_in, n_out, deg, mode)
    assert o.rel_l2(dC_a + dC_b, dC) <= 1e-4
    # linearity in dY (powers of two are exact through the fp16 scaling; a general factor rounds differently)
    dC_4 = ops.bwd_dcoeff(x, dy * 4.0, n_in, n_out, deg, mode)
    assert torch.equal(dC_4, 4.0 * dC)
    # a 32768-row block against the oracle
    blk = slice(300000, 300000 + 32768)
    _, dC_ref, _ = o.forward_backward(x[blk].cpu(), c_cpu, dy[blk].cpu(), need_dx=False)
    dC_blk = ops.bwd_dcoeff(x[blk].contiguous(), dy[blk].contiguous(), n_in, n_out, deg, mode)
    assert o.rel_l2(dC_blk.cpu(), dC_ref) <= TC_TOL
