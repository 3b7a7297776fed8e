"""GPU parity, fp32 FFMA mode: CUDA kernels through the C ABI vs the CPU oracle
and vs the reference's golden vectors.  Tolerance: rel-L2 <= 1e-5."""
import numpy as np
import pytest
import torch

import kan_b200
from kan_b200 import ops, workloads
from oracle import chebykan_oracle as o
from _util import FP32_TOL, OracleLayer, assert_guards_intact, guarded, make_case

pytestmark = pytest.mark.gpu

GOLDEN_CASES = ["tiny_d4", "mid_d8", "cfg1_shape", "deg32_uniform", "deg0", "deg1", "three_dim_input",
                "recurrence_path", "sparse_784", "wide_out", "kat_points"]

SHAPES = [
    # B, in, out, deg, dist
    (4096, 1024, 1024, 8, "normal"),     # configuration 3 at reduced batch
    (256, 784, 64, 4, "sparse"),         # configuration 2, first layer
    (256, 64, 10, 4, "normal"),          # configuration 2, second layer
    (4096, 64, 64, 32, "uniform3"),      # configuration 5 layer
    (1024, 2048, 2048, 4, "normal"),     # configuration 4 layer at reduced batch
    (127, 13, 7, 3, "normal"),
    (1, 5, 130, 2, "normal"),
    (100, 1, 1, 8, "normal"),
    (333, 17, 65, 16, "uniform3"),
    (64, 9, 3, 0, "normal"),
    (2500, 3, 2, 63, "normal"),
]


def run_all(x, coeffs, dy):
    n_in, n_out, dp1 = coeffs.shape
    xd, cd, dyd = x.cuda(), coeffs.cuda(), dy.cuda()
    packed = ops.pack_coeffs(cd, "fp32")
    y, yw = guarded((x.shape[0], n_out))
    ops.forward(xd, packed, n_in, n_out, dp1 - 1, "fp32", out=y)
    dC, dCw = guarded((n_in, n_out, dp1))
    ops.bwd_dcoeff(xd, dyd, n_in, n_out, dp1 - 1, "fp32", out=dC)
    dx, dxw = guarded(tuple(x.shape))
    ops.bwd_dx(xd, dyd, cd, "fp32", out=dx)
    torch.cuda.synchronize()
    assert_guards_intact(y, yw)
    assert_guards_intact(dC, dCw)
    assert_guards_intact(dx, dxw)
    return y.cpu(), dC.cpu(), dx.cpu()


@pytest.mark.parametrize("name", GOLDEN_CASES)
def test_golden_vectors(golden, name):
    c = golden[name]
    n_in = int(c["meta"][0])
    x = torch.from_numpy(c["x"]).reshape(-1, n_in).contiguous()
    y, dC, dx = run_all(x, torch.from_numpy(c["coeffs"]), torch.from_numpy(c["dy"]))
    assert o.rel_l2(y, c["y"]) <= FP32_TOL
    assert o.rel_l2(dC, c["dC"]) <= FP32_TOL
    if "dx" in c:
        assert o.rel_l2(dx.reshape(-1), c["dx"].reshape(-1)) <= FP32_TOL


@pytest.mark.parametrize("B,n_in,n_out,deg,dist", SHAPES)
def test_fwd_bwd_vs_oracle(B, n_in, n_out, deg, dist):
    x, coeffs, dy = make_case(B, n_in, n_out, deg, dist, seed=B + n_in + deg)
    y_ref, dC_ref, dx_ref = o.forward_backward(x, coeffs, dy)
    y, dC, dx = run_all(x, coeffs, dy)
    for name, got, ref in (("y", y, y_ref), ("dC", dC, dC_ref), ("dx", dx, dx_ref)):
        err = o.rel_l2(got, ref)
        if not err <= FP32_TOL:
            d = (got.double() - ref.double()).abs().reshape(got.shape[0], -1)
            r, c = divmod(int(d.argmax()), d.shape[1])
            pytest.fail(f"{name}: rel-L2 {err:.3e} > {FP32_TOL}; worst element [{r}, {c}]: "
                        f"{float(got.reshape(got.shape[0], -1)[r, c])!r} vs {float(ref.reshape(ref.shape[0], -1)[r, c])!r}; "
                        f"{int((d > 1e-3 * float(ref.abs().max())).sum())} elements off by more than 1e-3 of the largest value")


def test_bitwise_repeatable():
    x, coeffs, dy = make_case(1000, 96, 80, 8, seed=5)
    a = run_all(x, coeffs, dy)
    b = run_all(x, coeffs, dy)
    for u, v in zip(a, b):
        assert torch.equal(u, v)


# 128-row forward tiles: launch_fwd_ffma picks fwd_ffma_kernel<2,2> (outputs padded to a multiple of 128) or
# <2,1> (64-wide layers) once ceil(B/128) * column tiles reaches two CTAs per SM (296); every full-size fp32
# run uses them
LARGE_TILE_SHAPES = [
    (5000, 64, 1024, 2, "normal"),       # <2,2>: 40 x 8 tiles
    (6000, 1024, 1024, 8, "normal"),     # <2,2>: configuration 3's layer, ragged last row tile
    (2432, 2048, 2048, 4, "normal"),     # <2,2>: configuration 4's layer, 19 x 16 tiles
    (40000, 16, 64, 2, "normal"),        # <2,1>: 313 x 1 tiles
    (40000, 64, 64, 32, "uniform3"),     # <2,1>: configuration 5's layer
    (37999, 30, 70, 5, "normal"),        # <2,2> with ragged rows, inputs and outputs (70 -> 128 padded columns)
]


@pytest.mark.parametrize("B,n_in,n_out,deg,dist", LARGE_TILE_SHAPES)
def test_forward_128_row_tiles_vs_oracle(B, n_in, n_out, deg, dist):
    import math
    n_pad = math.ceil(n_out / 64) * 64
    col_tiles = n_pad // 128 if n_pad % 128 == 0 else n_pad // 64
    assert math.ceil(B / 128) * col_tiles >= 296, "shape no longer reaches the 128-row tiles"
    x, coeffs, _ = make_case(B, n_in, n_out, deg, dist, seed=B + n_in + deg)
    xd, cd = x.cuda(), coeffs.cuda()
    packed = ops.pack_coeffs(cd, "fp32")
    y, yw = guarded((B, n_out))
    ops.forward(xd, packed, n_in, n_out, deg, "fp32", out=y)
    torch.cuda.synchronize()
    assert_guards_intact(y, yw)
    assert o.rel_l2(y.cpu(), o.forward(x, coeffs)) <= FP32_TOL
    y2 = ops.forward(xd, packed, n_in, n_out, deg, "fp32")
    assert torch.equal(y, y2)


def _first_mismatch(name, a, b, tile_rows, tile_cols):
    """Where two runs of the same kernel differ: the message of the repeat test below."""
    diff = (a != b) & ~(torch.isnan(a) & torch.isnan(b))
    idx = diff.reshape(a.shape[0], -1).nonzero()
    r, c = int(idx[0, 0]), int(idx[0, 1])
    mx = float((a.double() - b.double()).abs().max())
    return (f"{name}: {int(diff.sum())} of {a.numel()} elements differ between two runs; first at [{r}, {c}] "
            f"(tile {r // tile_rows}, {c // tile_cols}): {float(a.reshape(a.shape[0], -1)[r, c])!r} vs "
            f"{float(b.reshape(a.shape[0], -1)[r, c])!r}; max abs difference {mx:.3e}")


# one launch plan per case: (4096, 1024, 1024, 8) = 1024 plain 64x64 forward tiles at two CTAs per SM, the dC kernel
# writing straight into dC (592 tiles, no batch split) and the 64-row dx tiles; (1024, 2048, 2048, 4) the same kernels on
# configuration 4's layer; (20000, 8, 8, 4) the batch-split dC path with its fixed-order reduction
@pytest.mark.parametrize("B,n_in,n_out,deg,reps", [(4096, 1024, 1024, 8, 40), (1024, 2048, 2048, 4, 10),
                                                   (20000, 8, 8, 4, 40), (6000, 1024, 1024, 8, 10)])
def test_fp32_kernels_repeat_bit_for_bit(B, n_in, n_out, deg, reps):
    """The fp32 kernels have a fixed summation order: `reps` runs in one process give identical bits."""
    x, coeffs, dy = make_case(B, n_in, n_out, deg, seed=B + n_in + deg)
    xd, cd, dyd = x.cuda(), coeffs.cuda(), dy.cuda()
    packed = ops.pack_coeffs(cd, "fp32")

    def run():
        y = torch.full((B, n_out), float("nan"), device="cuda")
        dC = torch.full((n_in, n_out, deg + 1), float("nan"), device="cuda")
        dx = torch.full((B, n_in), float("nan"), device="cuda")
        ops.forward(xd, packed, n_in, n_out, deg, "fp32", out=y)
        ops.bwd_dcoeff(xd, dyd, n_in, n_out, deg, "fp32", out=dC)
        ops.bwd_dx(xd, dyd, cd, "fp32", out=dx)
        return y, dC, dx

    first = run()
    y_ref, dC_ref, dx_ref = o.forward_backward(x, coeffs, dy)
    for name, got, ref in zip(("y", "dC", "dx"), first, (y_ref, dC_ref, dx_ref)):
        err = o.rel_l2(got.cpu(), ref)
        assert err <= FP32_TOL, f"{name}: rel-L2 {err:.3e} against the oracle"
    tiles = {"y": (64, 64), "dC": (128 // (deg + 1), 128 * (deg + 1)), "dx": (64, 128 // (deg + 1))}
    for rep in range(1, reps):
        again = run()
        for name, a, b in zip(("y", "dC", "dx"), first, again):
            if not torch.equal(a, b):
                pytest.fail(f"run {rep}: " + _first_mismatch(name, a, b, *tiles[name]))


def test_dcoeff_accumulate_and_split_batch():
    # large batch on a narrow layer forces the batch-split path and its workspace
    x, coeffs, dy = make_case(20000, 8, 8, 4, seed=9)
    _, dC_ref, _ = o.forward_backward(x, coeffs, dy, need_dx=False)
    assert _lib_ws(20000, 8, 8, 4) > 0
    xd, dyd = x.cuda(), dy.cuda()
    out = torch.ones(8, 8, 5, device="cuda")
    ops.bwd_dcoeff(xd, dyd, 8, 8, 4, "fp32", out=out, accumulate=True)
    assert o.rel_l2(out.cpu() - 1.0, dC_ref) <= 2e-5       # "+1" costs a few ulps of the sum
    out2 = ops.bwd_dcoeff(xd, dyd, 8, 8, 4, "fp32")
    assert o.rel_l2(out2.cpu(), dC_ref) <= FP32_TOL
    # direct (single split) accumulate path
    x, coeffs, dy = make_case(64, 300, 200, 4, seed=10)
    _, dC_ref, _ = o.forward_backward(x, coeffs, dy, need_dx=False)
    assert _lib_ws(64, 300, 200, 4) == 0
    out = torch.zeros(300, 200, 5, device="cuda")
    ops.bwd_dcoeff(x.cuda(), dy.cuda(), 300, 200, 4, "fp32", out=out, accumulate=True)
    ops.bwd_dcoeff(x.cuda(), dy.cuda(), 300, 200, 4, "fp32", out=out, accumulate=True)
    assert o.rel_l2(out.cpu(), 2 * dC_ref) <= FP32_TOL


def _lib_ws(B, n_in, n_out, deg):
    from kan_b200 import _lib
    return _lib.load().chebykan_workspace_bytes(_lib.OP_BWD_DCOEFF, B, n_in, n_out, deg, 0)


def test_known_answers_on_gpu():
    layer = kan_b200.ChebyKANLayer(1, 1, 4).cuda()
    with torch.no_grad():
        layer.cheby_coeffs.fill_(1.0)
    x = torch.tensor([[0.0], [20.0], [-20.0]], device="cuda")
    y = layer(x).cpu().flatten()
    # sum_d T_d: x=0 -> 1+0-1+0+1 = 1; t=+1 -> 5; t=-1 -> 1-1+1-1+1 = 1
    assert torch.allclose(y, torch.tensor([1.0, 5.0, 1.0]), atol=1e-6)
    # degree 0: y = sum_i C[i,o,0] for every row
    l0 = kan_b200.ChebyKANLayer(7, 3, 0).cuda()
    y0 = l0(torch.randn(11, 7, device="cuda"))
    assert torch.allclose(y0, l0.cheby_coeffs[:, :, 0].sum(0).expand(11, 3), atol=1e-7)


def test_saturated_tanh_gives_zero_dx_not_nan():
    """Documented departure: the reference's autograd yields NaN where tanh(x) == +-1."""
    x = torch.tensor([[12.0, 0.3], [-15.0, 9.0]])
    coeffs = torch.randn(2, 2, 5)
    dy = torch.ones(2, 2)
    _, _, dx_ref = o.forward_backward(x, coeffs, dy)
    dx = ops.bwd_dx(x.cuda(), dy.cuda(), coeffs.cuda(), "fp32").cpu()
    assert torch.isnan(dx_ref[0, 0]) and torch.isnan(dx_ref[1, 0])
    assert dx[0, 0] == 0 and dx[1, 0] == 0
    finite = torch.isfinite(dx_ref)
    assert o.rel_l2(dx[finite], dx_ref[finite]) <= FP32_TOL


def test_empty_batch_and_flatten_rule():
    layer = kan_b200.ChebyKANLayer(4, 3, 3).cuda()
    y = layer(torch.empty(0, 4, device="cuda"))
    assert y.shape == (0, 3)
    y = layer(torch.randn(2, 5, 4, device="cuda"))
    assert y.shape == (10, 3)                     # leading dimensions are flattened, not restored
    with pytest.raises(RuntimeError):
        layer(torch.randn(2, 4, 5, device="cuda").transpose(1, 2))   # leading dims cannot be merged: view fails
    # a non-contiguous input whose view succeeds is accepted, as in the reference
    xt = torch.randn(4, 6, device="cuda").t()
    assert o.rel_l2(layer(xt).detach().cpu(), o.forward(xt.cpu().contiguous(), layer.cheby_coeffs.detach().cpu())) <= FP32_TOL
    with pytest.raises(RuntimeError, match="Float"):
        layer(torch.randn(6, 4, device="cuda", dtype=torch.float64))


def test_unaligned_view_input_is_accepted():
    """A contiguous view that starts in the middle of a buffer (not 16-byte aligned) works like in the reference."""
    torch.manual_seed(8)
    layer = kan_b200.ChebyKANLayer(5, 6, 3).cuda()
    base = torch.randn(1 + 40 * 5, device="cuda")
    x = base[1:].view(40, 5).requires_grad_(True)          # data_ptr is 4 bytes past an aligned address
    assert x.data_ptr() % 16 != 0
    y = layer(x)
    y.sum().backward()
    y_ref, dC_ref, dx_ref = o.forward_backward(x.detach().cpu(), layer.cheby_coeffs.detach().cpu(), torch.ones(40, 6))
    assert o.rel_l2(y.detach().cpu(), y_ref) <= FP32_TOL
    assert o.rel_l2(x.grad.cpu(), dx_ref) <= FP32_TOL
    assert o.rel_l2(layer.cheby_coeffs.grad.cpu(), dC_ref) <= FP32_TOL


def test_c_abi_rejects_bad_arguments():
    from kan_b200 import _lib
    lib = _lib.load()
    buf = torch.zeros(1024, device="cuda")
    st = ops.status_tensor("cuda")
    p = buf.data_ptr()
    assert lib.chebykan_fwd(p + 4, p, p, 4, 4, 4, 2, 0, st.data_ptr(), None) == -2     # misaligned
    assert lib.chebykan_fwd(p, p, p, 4, 0, 4, 2, 0, st.data_ptr(), None) == -1         # in = 0
    assert lib.chebykan_fwd(p, p, p, 4, 4, 4, 2, 9, st.data_ptr(), None) == -1         # bad mode
    assert lib.chebykan_fwd(None, p, p, 4, 4, 4, 2, 0, st.data_ptr(), None) == -1      # null x
    assert lib.chebykan_bwd_dcoeff(p, p, p, None, 0, 1 << 20, 8, 8, 4, 0, 0, None, None) == -6  # no workspace
    assert lib.chebykan_adam_step(p, p, p, p, 16, 0.1, 0.9, 0.999, 1e-8, 0, 1.0, None) == -1   # step < 1
    assert lib.chebykan_bwd_dx(p, p, p, p, None, 0, 64, 8, 8, 3, 1, st.data_ptr(), None) == -6   # tf32 dx: no workspace
    torch.cuda.synchronize()


def test_layer_autograd_two_layer_model():
    """Configuration 2 (784->64->LN->10, degree 4, batch 256, cross-entropy): gradients of every parameter."""
    cfg = workloads.CONFIGS["cfg2"]
    x, labels = workloads.make_inputs(cfg)
    ref = workloads.build_model(cfg, OracleLayer)
    ours = workloads.build_model(cfg, kan_b200.ChebyKANLayer)
    for a, b in zip(ref.parameters(), ours.parameters()):
        assert torch.equal(a, b)                      # same seed, same CPU RNG stream
    ours = ours.cuda()
    loss_ref = torch.nn.functional.cross_entropy(ref(x), labels)
    loss_ref.backward()
    loss = torch.nn.functional.cross_entropy(ours(x.cuda()), labels.cuda())
    loss.backward()
    assert abs(float(loss.detach()) - float(loss_ref.detach())) <= 1e-5 * abs(float(loss_ref.detach()))
    for (n, a), (_, b) in zip(ref.named_parameters(), ours.named_parameters()):
        assert o.rel_l2(b.grad.cpu(), a.grad) <= 2e-5, n


@pytest.mark.parametrize("opt_name", ["sgd", "adam"])
def test_optimizer_steps_vs_torch(opt_name):
    torch.manual_seed(3)
    p_ref = torch.randn(1000 + 3).requires_grad_(True)        # odd length exercises the scalar tail
    p = p_ref.detach().clone().cuda().requires_grad_(True)
    if opt_name == "sgd":
        ref_opt = torch.optim.SGD([p_ref], lr=1e-2)
        opt = kan_b200.optim.SGD([p], lr=1e-2)
    else:
        ref_opt = torch.optim.Adam([p_ref], lr=1e-3)
        opt = kan_b200.optim.Adam([p], lr=1e-3)
    for step in range(20):
        g = torch.randn(1003)
        p_ref.grad = g.clone()
        p.grad = g.cuda()
        ref_opt.step()
        opt.step()
    assert o.rel_l2(p.detach().cpu(), p_ref.detach()) <= FP32_TOL


def test_training_loop_config1(golden):
    """README loop: 1 -> 1, degree 8, 100 points, MSE, Adam(0.01), 1000 steps, from the reference's weights."""
    layer = kan_b200.ChebyKANLayer(1, 1, 8)
    with torch.no_grad():
        layer.cheby_coeffs.copy_(torch.from_numpy(golden["cfg1_train"]["init_coeffs"]))
    layer = layer.cuda()
    x, tgt = workloads.make_inputs(workloads.CONFIGS["cfg1"])
    x, tgt = x.cuda(), tgt.cuda()
    opt = kan_b200.optim.Adam(layer.parameters(), lr=0.01)
    got = []
    for step in range(1000):
        opt.zero_grad()
        loss = torch.nn.functional.mse_loss(layer(x), tgt)
        loss.backward()
        opt.step()
        if step in (0, 99, 499, 999):
            got.append(float(loss.detach()))
    assert np.allclose(got, golden["cfg1_train"]["losses"], rtol=2e-3)
    assert o.rel_l2(layer.cheby_coeffs.detach().cpu(), golden["cfg1_train"]["final_coeffs"]) <= 2e-3


def test_forward_through_host_buffers():
    x, coeffs, _ = make_case(777, 24, 40, 6, seed=21)
    y_ref = o.forward(x, coeffs)
    y, _ = ops.forward_host(x.pin_memory(), coeffs, "fp32")
    assert o.rel_l2(y, y_ref) <= FP32_TOL


def test_graphed_training_step_config1(golden):
    """The README loop replayed as one CUDA graph per step (capturable Adam): same loss curve and final coefficients."""
    layer = kan_b200.ChebyKANLayer(1, 1, 8)
    with torch.no_grad():
        layer.cheby_coeffs.copy_(torch.from_numpy(golden["cfg1_train"]["init_coeffs"]))
    layer = layer.cuda()
    x, tgt = workloads.make_inputs(workloads.CONFIGS["cfg1"])
    x, tgt = x.cuda(), tgt.cuda()
    opt = kan_b200.optim.Adam(layer.parameters(), lr=0.01, capturable=True)
    # the constructor runs 3 eager warm-up steps and 1 capture step: restore the start state afterwards
    step = kan_b200.graph.GraphedTrainStep(layer, torch.nn.functional.mse_loss, opt, x, tgt)
    with torch.no_grad():
        layer.cheby_coeffs.copy_(torch.from_numpy(golden["cfg1_train"]["init_coeffs"]).cuda())
    for st in opt.state.values():
        st["exp_avg"].zero_(); st["exp_avg_sq"].zero_(); st["step_dev"].zero_()
    got = []
    for i in range(1000):
        loss = step()
        if i in (0, 99, 499, 999):
            got.append(float(loss.detach()))
    assert np.allclose(got, golden["cfg1_train"]["losses"], rtol=2e-3)
    assert o.rel_l2(layer.cheby_coeffs.detach().cpu(), golden["cfg1_train"]["final_coeffs"]) <= 2e-3
    assert int(next(iter(opt.state.values()))["step_dev"].item()) == 1000
    with pytest.raises(ValueError):
        kan_b200.graph.GraphedTrainStep(layer, torch.nn.functional.mse_loss,
                                        kan_b200.optim.Adam(layer.parameters(), lr=0.01), x, tgt)


def test_fused_single_launch_step_config1(golden):
    """The README loop with the whole step (forward, MSE, backward, Adam) as one kernel launch: the reference's loss
    curve and final coefficients; one step equals the staged kernels' step; bitwise repeatable."""
    layer = kan_b200.ChebyKANLayer(1, 1, 8)
    with torch.no_grad():
        layer.cheby_coeffs.copy_(torch.from_numpy(golden["cfg1_train"]["init_coeffs"]))
    layer = layer.cuda()
    x, tgt = workloads.make_inputs(workloads.CONFIGS["cfg1"])
    x, tgt = x.cuda(), tgt.cuda()
    step = kan_b200.small.FusedTrainStep(layer, "adam", lr=0.01)
    got = []
    for i in range(1000):
        loss = step(x, tgt)
        if i in (0, 99, 499, 999):
            got.append(float(loss))
    assert np.allclose(got, golden["cfg1_train"]["losses"], rtol=2e-3)
    assert o.rel_l2(layer.cheby_coeffs.detach().cpu(), golden["cfg1_train"]["final_coeffs"]) <= 2e-3
    assert int(step.step_count.item()) == 1000
    # an eager forward after the fused steps sees the updated coefficients (the packed copy is refreshed)
    assert o.rel_l2(layer(x).detach().cpu(), o.forward(x.cpu(), layer.cheby_coeffs.detach().cpu())) <= FP32_TOL


@pytest.mark.parametrize("opt_name", ["adam", "sgd"])
@pytest.mark.parametrize("shape", [(100, 1, 1, 8), (333, 5, 3, 4), (1, 2, 16, 0), (2000, 8, 16, 3), (64, 16, 4, 31)])
def test_fused_single_launch_step_matches_oracle(opt_name, shape):
    B, n_in, n_out, deg = shape
    g = torch.Generator().manual_seed(B + deg)
    x = torch.randn(B, n_in, generator=g)
    tgt = torch.randn(B, n_out, generator=g)
    torch.manual_seed(B)
    layer = kan_b200.ChebyKANLayer(n_in, n_out, deg).cuda()
    c0 = layer.cheby_coeffs.detach().cpu().clone()
    step = kan_b200.small.FusedTrainStep(layer, opt_name, lr=0.05, keep_grad=True)
    ref_p = c0.clone().requires_grad_(True)
    ref_opt = (torch.optim.Adam([ref_p], lr=0.05) if opt_name == "adam" else torch.optim.SGD([ref_p], lr=0.05))
    for _ in range(3):
        loss = step(x.cuda(), tgt.cuda())
        ref_opt.zero_grad()
        ref_loss = torch.nn.functional.mse_loss(o.forward(x, ref_p), tgt)
        ref_loss.backward()
        assert abs(float(loss) - float(ref_loss)) <= 2e-5 * abs(float(ref_loss))
        assert o.rel_l2(layer.cheby_coeffs.grad.cpu(), ref_p.grad) <= FP32_TOL
        ref_opt.step()
    # Adam divides by sqrt(v) + eps: where a gradient is almost zero the update direction is ill-conditioned
    assert o.rel_l2(layer.cheby_coeffs.detach().cpu() - c0, ref_p.detach() - c0) <= (1e-3 if opt_name == "adam" else 1e-5)
    # bitwise repeatable: the same three steps from the same start give the same bits
    layer2 = kan_b200.ChebyKANLayer(n_in, n_out, deg).cuda()
    with torch.no_grad():
        layer2.cheby_coeffs.copy_(c0.cuda())
    step2 = kan_b200.small.FusedTrainStep(layer2, opt_name, lr=0.05)
    for _ in range(3):
        step2(x.cuda(), tgt.cuda())
    assert torch.equal(layer2.cheby_coeffs.detach(), layer.cheby_coeffs.detach())


def test_fused_single_launch_step_limits():
    assert kan_b200.small.supported(100, 1, 1, 8) and kan_b200.small.supported(3072, 8, 8, 3)
    assert not kan_b200.small.supported(100, 64, 64, 8)          # 36864 coefficients
    assert not kan_b200.small.supported(100, 4, 17, 2)           # more than 16 outputs
    assert not kan_b200.small.supported(50000, 1, 1, 8)          # rows do not fit shared memory
    layer = kan_b200.ChebyKANLayer(64, 64, 8).cuda()
    with pytest.raises(RuntimeError, match="does not cover"):
        kan_b200.small.FusedTrainStep(layer)(torch.randn(10, 64).cuda(), torch.randn(10, 64).cuda())
    with pytest.raises(RuntimeError, match="CUDA"):
        kan_b200.small.FusedTrainStep(kan_b200.ChebyKANLayer(1, 1, 2))
    with pytest.raises(ValueError):
        kan_b200.small.FusedTrainStep(layer, optimizer="lbfgs")


def test_graphed_step_equals_eager_config2():
    cfg = workloads.CONFIGS["cfg2"]
    x, labels = workloads.make_inputs(cfg)
    x, labels = x.cuda(), labels.cuda()
    eager = workloads.build_model(cfg, kan_b200.ChebyKANLayer).cuda()
    graphed_model = workloads.build_model(cfg, kan_b200.ChebyKANLayer).cuda()
    opt_e = kan_b200.optim.Adam(eager.parameters(), lr=1e-3)
    opt_g = kan_b200.optim.Adam(graphed_model.parameters(), lr=1e-3, capturable=True)
    step = kan_b200.graph.GraphedTrainStep(graphed_model, torch.nn.functional.cross_entropy, opt_g, x, labels)
    n_done = 3                                           # 3 eager warm-up steps; capturing records, it does not run
    for _ in range(6):
        step()
        n_done += 1
    for _ in range(n_done):
        opt_e.zero_grad()
        torch.nn.functional.cross_entropy(eager(x), labels).backward()
        opt_e.step()
    for a, b in zip(eager.parameters(), graphed_model.parameters()):
        assert o.rel_l2(b.detach().cpu(), a.detach().cpu()) <= 1e-5


@pytest.mark.parametrize("B,n_in,n_out,deg", [(33, 7, 5, 8), (100, 1, 1, 8), (16, 40, 12, 3), (9, 3, 2, 32), (5, 4, 4, 0)])
def test_jacobian_matches_autograd(B, n_in, n_out, deg):
    """layer.jacobian returns d y / d x of the oracle (autograd on the CPU), shape [B, out, in]."""
    torch.manual_seed(B + deg)
    layer = kan_b200.ChebyKANLayer(n_in, n_out, deg, init_scale=0.3).cuda()
    x = torch.randn(B, n_in)
    J = layer.jacobian(x.cuda()).cpu()
    assert J.shape == (B, n_out, n_in)
    c = layer.cheby_coeffs.detach().cpu()
    xr = x.clone().requires_grad_(True)
    y = o.forward(xr, c)
    J_ref = torch.stack([torch.autograd.grad(y[:, k].sum(), xr, retain_graph=True)[0] for k in range(n_out)], 1)
    assert o.rel_l2(J, J_ref) <= FP32_TOL
    assert o.rel_l2(layer.compute_derivatives(x.cuda()).cpu(), J_ref.sum(-1)) <= FP32_TOL
    with pytest.raises(NotImplementedError):
        layer.compute_derivatives(x.cuda(), order=2)


@pytest.mark.parametrize("B,n_in,n_out,deg", [(256, 784, 64, 4), (64, 200, 10, 8), (100, 1024, 130, 3), (1, 64, 64, 5)])
def test_small_batch_forward_splits_the_contraction_over_a_cluster(B, n_in, n_out, deg):
    """Few row tiles and many inputs: the fp32 forward runs one cluster of 2-8 CTAs per tile and adds the partial
    tiles through distributed shared memory in rank order: within tolerance of the oracle and bitwise repeatable."""
    x, coeffs, _ = make_case(B, n_in, n_out, deg, seed=B + n_in)
    xd, cd = x.cuda(), coeffs.cuda()
    packed = ops.pack_coeffs(cd, "fp32")
    y, yw = guarded((B, n_out))
    ops.forward(xd, packed, n_in, n_out, deg, "fp32", out=y)
    torch.cuda.synchronize()
    assert_guards_intact(y, yw)
    assert o.rel_l2(y.cpu(), o.forward(x, coeffs)) <= FP32_TOL
    y2 = ops.forward(xd, packed, n_in, n_out, deg, "fp32")
    assert torch.equal(y, y2)
