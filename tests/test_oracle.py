"""CPU tests of the oracle: against the unmodified reference (when its tree is
present), against the committed golden vectors, and against known answers."""
import numpy as np
import pytest
import torch

from oracle import chebykan_oracle as o
from oracle import ref_loader

CASE_NAMES = ["tiny_d4", "mid_d8", "cfg1_shape", "deg32_uniform", "deg0", "deg1", "three_dim_input",
              "recurrence_path", "sparse_784", "wide_out", "kat_points"]


@pytest.mark.parametrize("name", CASE_NAMES)
def test_oracle_matches_golden(golden, name):
    """The restatement reproduces the reference's stored outputs (same ATen CPU ops)."""
    c = golden[name]
    n_in, n_out, deg, rec = [int(v) for v in c["meta"]]
    x = torch.from_numpy(c["x"])
    coeffs = torch.from_numpy(c["coeffs"])
    dy = torch.from_numpy(c["dy"])
    y, dC, dx = o.forward_backward(x, coeffs, dy, use_recurrence=bool(rec), need_dx=not rec)
    # bit-exact on the machine that generated the fixtures; other CPUs may pick other
    # vector kernels, so allow rounding-level differences
    assert o.rel_l2(y, c["y"]) <= 2e-6
    assert o.rel_l2(dC, c["dC"]) <= 2e-6
    if not rec:
        assert o.rel_l2(dx.reshape(-1), c["dx"].reshape(-1)) <= 2e-6
    assert y.shape == (x.numel() // n_in, n_out)


@pytest.mark.skipif(not ref_loader.available(), reason="reference tree not on this machine")
@pytest.mark.parametrize("shape,n_in,n_out,deg", [((50,), 8, 6, 8), ((3, 7), 5, 4, 3), ((64,), 64, 64, 32),
                                                 ((10,), 3, 2, 0)])
def test_oracle_bit_exact_vs_reference(shape, n_in, n_out, deg):
    Ref = ref_loader.reference_layer_cls()
    torch.manual_seed(11)
    layer = Ref(n_in, n_out, deg)
    torch.manual_seed(11)
    coeffs = o.init_coeffs(n_in, n_out, deg)
    assert torch.equal(layer.cheby_coeffs.detach(), coeffs)      # same RNG consumption
    x = torch.randn(*shape, n_in, requires_grad=True)
    y = layer(x)
    dy = torch.randn_like(y)
    y.backward(dy)
    y2, dC2, dx2 = o.forward_backward(x.detach(), coeffs, dy)
    assert torch.equal(y.detach(), y2)
    assert torch.equal(layer.cheby_coeffs.grad, dC2)
    assert torch.equal(x.grad, dx2)


@pytest.mark.skipif(not ref_loader.available(), reason="reference tree not on this machine")
def test_recurrence_path_bit_exact_vs_reference():
    Ref = ref_loader.reference_layer_cls()
    torch.manual_seed(5)
    layer = Ref(6, 4, 8, use_recurrence=True)
    x = torch.randn(31, 6)
    assert torch.equal(layer(x).detach(), o.forward(x, layer.cheby_coeffs.detach(), use_recurrence=True))


def test_init_scale_is_a_std():
    torch.manual_seed(0)
    c = o.init_coeffs(64, 64, 8)
    assert abs(float(c.std()) - 1.0 / (64 * 9)) < 2e-5
    torch.manual_seed(0)
    c0 = o.init_coeffs(64, 64, 8, init_scale=0.0)     # falsy 0 selects the default
    assert torch.equal(c, c0)


def test_known_answers():
    # x = 0 -> T_d(0) = cos(d pi/2); x -> +inf: all ones; x -> -inf: (-1)^d
    t = torch.tensor([[0.0], [1.0], [-1.0]])
    phi = o.basis_closed_form(t, 4)
    assert torch.allclose(phi[0, 0], torch.tensor([1.0, 0.0, -1.0, 0.0, 1.0]), atol=1e-6)
    assert torch.allclose(phi[1, 0], torch.ones(5), atol=1e-6)
    assert torch.allclose(phi[2, 0], torch.tensor([1.0, -1.0, 1.0, -1.0, 1.0]), atol=1e-6)
    # degree 0: y = sum_i C[i,o,0]
    c = torch.randn(3, 2, 1)
    y = o.forward(torch.randn(5, 3), c)
    assert torch.allclose(y, c[:, :, 0].sum(0).expand(5, 2), atol=1e-6)
    # one-hot coefficients select a single T_d(tanh x_i)
    c = torch.zeros(3, 2, 5)
    c[1, 0, 3] = 1.0
    x = torch.randn(7, 3)
    t1 = torch.tanh(x[:, 1])
    assert torch.allclose(o.forward(x, c)[:, 0], 4 * t1 ** 3 - 3 * t1, atol=1e-5)


def test_closed_form_vs_recurrence_and_f64():
    g = torch.Generator().manual_seed(3)
    x = torch.rand(512, 16, generator=g) * 6 - 3
    c = torch.randn(16, 8, 33, generator=g) / (16 * 33)
    dy = torch.randn(512, 8, generator=g)
    y, dC, dx = o.forward_backward(x, c, dy)
    y_r = o.forward(x, c, use_recurrence=True)
    y64, dC64, dx64 = o.analytic_f64(x.numpy(), c.numpy(), dy.numpy())
    assert o.rel_l2(y_r, y) < 5e-6
    assert o.rel_l2(y, y64) < 5e-6 and o.rel_l2(dC, dC64) < 5e-6 and o.rel_l2(dx, dx64) < 5e-6


def test_dx_is_nan_where_tanh_saturates():
    """Reference semantics the CUDA path deliberately departs from: autograd gives NaN at t = +-1."""
    x = torch.tensor([[12.0, 0.3]])
    c = torch.randn(2, 2, 4)
    _, _, dx = o.forward_backward(x, c, torch.ones(1, 2))
    assert torch.isnan(dx[0, 0]) and torch.isfinite(dx[0, 1])


def test_optimizer_restatement_matches_torch():
    torch.manual_seed(1)
    p = torch.randn(50)
    ref = p.clone().requires_grad_(True)
    opt = torch.optim.Adam([ref], lr=0.01)
    m = torch.zeros(50)
    v = torch.zeros(50)
    for step in range(1, 6):
        g = torch.randn(50)
        ref.grad = g.clone()
        opt.step()
        p, m, v = o.adam_step(p, g, m, v, step, 0.01)
    assert o.rel_l2(p, ref.detach()) < 1e-6
    q = torch.randn(10)
    rq = q.clone().requires_grad_(True)
    sgd = torch.optim.SGD([rq], lr=0.1)
    g = torch.randn(10)
    rq.grad = g.clone()
    sgd.step()
    assert torch.allclose(o.sgd_step(q, g, 0.1), rq.detach())


def test_cfg1_loss_curve(golden):
    """README training loop: the oracle reproduces the reference's loss trajectory."""
    init = torch.from_numpy(golden["cfg1_train"]["init_coeffs"]).clone().requires_grad_(True)
    xs = torch.linspace(-1, 1, 100, dtype=torch.float64).float().view(100, 1)
    tgt = torch.sin(2 * np.pi * xs)
    opt = torch.optim.Adam([init], lr=0.01)
    got = []
    for step in range(1000):
        opt.zero_grad()
        loss = torch.nn.functional.mse_loss(o.forward(xs, init), tgt)
        loss.backward()
        opt.step()
        if step in (0, 99, 499, 999):
            got.append(float(loss.detach()))
    assert np.allclose(got, golden["cfg1_train"]["losses"], rtol=1e-3)
