"""GPU parity of the Jacobi and Hermite layers (the fp32 kernels with a table-driven recurrence) against the CPU
oracle of the reference's layers, against the reference's golden vectors, and through the drop-in layer classes."""
import copy

import pytest
import torch

import kan_b200
from kan_b200 import ops
from oracle import chebykan_oracle as o
from oracle import polykan_oracle as po
from conftest import load_golden_poly
from _util import FP32_TOL, TC_TOL, guarded, assert_guards_intact

pytestmark = pytest.mark.gpu

GOLDEN_NAMES = sorted(load_golden_poly())


def lib_family(fam: dict):
    """The library's description of an oracle family dictionary."""
    if fam["kind"] == "jacobi":
        return ops.make_family("jacobi", alpha=fam.get("alpha", 0.0), beta=fam.get("beta", 0.0))
    kind = "hermite" if fam.get("scaling", "physicist") == "physicist" else "hermite_prob"
    dom = fam.get("domain")
    if dom is not None and fam.get("normalize_domain", True):
        return ops.make_family(kind, scale=6.0 / (dom[1] - dom[0]), affine=True, shift=dom[0], offset=-3.0)
    return ops.make_family(kind)


def run_all(fam: dict, x, coeffs, dy):
    lf = lib_family(fam)
    n_in, n_out, dp1 = coeffs.shape
    xd, cd, dyd = x.cuda(), coeffs.cuda(), dy.cuda()
    y, y_whole = guarded((x.shape[0], n_out))
    dC, dC_whole = guarded(tuple(coeffs.shape))
    dx, dx_whole = guarded(tuple(x.shape))
    ops.family_forward(lf, xd, ops.pack_coeffs(cd, "fp32"), n_in, n_out, dp1 - 1, "fp32", out=y)
    ops.family_bwd_dcoeff(lf, xd, dyd, n_in, n_out, dp1 - 1, out=dC)
    ops.family_bwd_dx(lf, xd, dyd, cd, out=dx)
    torch.cuda.synchronize()
    for v, w in ((y, y_whole), (dC, dC_whole), (dx, dx_whole)):
        assert_guards_intact(v, w)
    return y.cpu(), dC.cpu(), dx.cpu()


@pytest.mark.parametrize("name", GOLDEN_NAMES)
def test_kernels_match_reference_golden(golden_poly, name):
    c = golden_poly[name]
    x, coeffs, dy = (torch.from_numpy(c[k]) for k in ("x", "coeffs", "dy"))
    y, dC, dx = run_all(c["family"], x, coeffs, dy)
    assert o.rel_l2(y, c["y"]) <= FP32_TOL
    assert o.rel_l2(dC, c["dC"]) <= FP32_TOL
    if c["dx"].any():
        assert o.rel_l2(dx, c["dx"]) <= FP32_TOL
    else:
        assert not bool(dx.any())


FAMILIES = [
    {"kind": "jacobi"},
    {"kind": "jacobi", "alpha": 0.5, "beta": -0.3},
    {"kind": "jacobi", "alpha": 2.0, "beta": 1.0},
    {"kind": "hermite"},
    {"kind": "hermite", "scaling": "probabilist"},
    {"kind": "hermite", "domain": (-4.0, 4.0)},
]
# (rows, in, out, degree): ragged edges, the 128-row tile variants (2,1) and (2,2), the cluster-split small batch,
# one input, one output, degree 0/1, a degree-32 contraction
SHAPES = [(257, 33, 17, 5), (40000, 24, 40, 4), (20000, 16, 130, 3), (64, 512, 32, 6), (1, 1, 1, 8), (77, 3, 2, 0),
          (77, 3, 2, 1), (513, 9, 70, 32), (4096, 64, 64, 12)]


@pytest.mark.parametrize("fam", FAMILIES, ids=lambda f: "-".join(str(v) for v in f.values()))
@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_kernels_match_oracle(fam, shape):
    B, n_in, n_out, deg = shape
    if fam["kind"] == "hermite" and deg > 16:
        # H_32(3) ~ 1e21 against H_0 = 1: the columns of one basis row span more than fp32 can add up, in the
        # reference as much as here; the Hermite layers are checked up to degree 12
        pytest.skip("Hermite columns of this degree exceed fp32's dynamic range within one row")
    g = torch.Generator().manual_seed(B + n_in + deg)
    x = torch.randn(B, n_in, generator=g)
    if fam.get("domain"):
        x = x.clamp(-4, 4)
    coeffs = torch.randn(n_in, n_out, deg + 1, generator=g) / (n_in * (deg + 1))
    dy = torch.randn(B, n_out, generator=g)
    y_ref, dC_ref, dx_ref = po.forward_backward(fam, x, coeffs, dy)
    y, dC, dx = run_all(fam, x, coeffs, dy)
    assert o.rel_l2(y, y_ref) <= FP32_TOL
    assert o.rel_l2(dC, dC_ref) <= FP32_TOL
    if deg > 0:
        assert o.rel_l2(dx, dx_ref) <= FP32_TOL
    else:
        assert not bool(dx.any())


# (rows, in, out, degree): CTA pairs on 2 x 256-output tiles, a single 256-wide tile, 128- and 64-wide tiles, an input
# count that rules out the TMA path for x, ragged everything, one row
TC_SHAPES = [(1000, 96, 520, 5), (300, 64, 256, 4), (257, 40, 100, 8), (4096, 64, 64, 12), (333, 33, 17, 5),
             (1, 8, 600, 3), (128, 256, 1024, 0), (64, 70, 390, 1)]


@pytest.mark.parametrize("mode", ["bf16", "tf32"])
@pytest.mark.parametrize("fam", FAMILIES, ids=lambda f: "-".join(str(v) for v in f.values()))
@pytest.mark.parametrize("shape", TC_SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_tensor_core_forward_matches_oracle(mode, fam, shape):
    B, n_in, n_out, deg = shape
    g = torch.Generator().manual_seed(B + n_in + deg + 1)
    x = torch.randn(B, n_in, generator=g)
    if fam.get("domain"):
        x = x.clamp(-4, 4)
    coeffs = torch.randn(n_in, n_out, deg + 1, generator=g) / (n_in * (deg + 1))
    y, whole = guarded((B, n_out))
    ops.family_forward(lib_family(fam), x.cuda(), ops.pack_coeffs(coeffs.cuda(), mode), n_in, n_out, deg, mode, out=y)
    torch.cuda.synchronize()
    ops.check_status()
    assert_guards_intact(y, whole)
    # bf16 mode stores the coefficients in bf16: the oracle evaluates with the same rounded values
    y_ref = po.forward(fam, x, coeffs.bfloat16().float() if mode == "bf16" else coeffs)
    assert o.rel_l2(y.cpu(), y_ref) <= TC_TOL


# backward on the tensor cores (kind::tf32 in both modes): CTA pairs and single CTAs, ragged tiles, narrow and wide
# outputs (narrow layers must not take the Chebyshev-only fp16-operand kernel), degree 0 and 1, one row
TC_BWD_SHAPES = [(1000, 96, 520, 5), (300, 64, 256, 4), (4096, 64, 64, 12), (257, 40, 100, 8), (64, 72, 392, 1),
                 (128, 256, 1024, 0), (1, 8, 600, 3), (5000, 33, 20, 6)]


@pytest.mark.parametrize("fam", FAMILIES, ids=lambda f: "-".join(str(v) for v in f.values()))
@pytest.mark.parametrize("shape", TC_BWD_SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_tensor_core_backward_matches_oracle(fam, shape):
    B, n_in, n_out, deg = shape
    g = torch.Generator().manual_seed(B + n_in + deg + 2)
    x = torch.randn(B, n_in, generator=g)
    if fam.get("domain"):
        x = x.clamp(-4, 4)
    coeffs = torch.randn(n_in, n_out, deg + 1, generator=g) / (n_in * (deg + 1))
    dy = torch.randn(B, n_out, generator=g)
    _, dC_ref, dx_ref = po.forward_backward(fam, x, coeffs, dy)
    lf = lib_family(fam)
    dC, dC_whole = guarded(tuple(coeffs.shape))
    dx, dx_whole = guarded(tuple(x.shape))
    ops.family_bwd_dcoeff(lf, x.cuda(), dy.cuda(), n_in, n_out, deg, "tf32", out=dC)
    ops.family_bwd_dx(lf, x.cuda(), dy.cuda(), coeffs.cuda(), "tf32", out=dx)
    torch.cuda.synchronize()
    ops.check_status()
    assert_guards_intact(dC, dC_whole)
    assert_guards_intact(dx, dx_whole)
    assert o.rel_l2(dC.cpu(), dC_ref) <= TC_TOL
    if deg > 0:
        assert o.rel_l2(dx.cpu(), dx_ref) <= TC_TOL
    else:
        assert not bool(dx.any())
    # accumulate adds into what is there
    acc = ops.family_bwd_dcoeff(lf, x.cuda(), dy.cuda(), n_in, n_out, deg, "bf16", out=dC.clone(), accumulate=True)
    assert o.rel_l2(acc.cpu(), 2 * dC_ref) <= TC_TOL


@pytest.mark.parametrize("mode", ["bf16", "tf32"])
def test_tensor_core_layers_train_on_the_tensor_cores(mode):
    torch.manual_seed(4)
    layer = kan_b200.JacobiKANLayer(48, 300, 6, alpha=0.5, beta=-0.3, math_mode=mode).cuda()
    coeffs = layer.jacobi_coeffs.detach().cpu()
    x = torch.randn(700, 48)
    dy = torch.randn(700, 300)
    xd = x.cuda().requires_grad_(True)
    y = layer(xd)
    y.backward(dy.cuda())
    ops.check_status()
    fam = {"kind": "jacobi", "alpha": 0.5, "beta": -0.3}
    y_ref, dC_ref, dx_ref = po.forward_backward(fam, x, coeffs, dy)
    assert o.rel_l2(y.detach().cpu(), po.forward(fam, x, coeffs.bfloat16().float() if mode == "bf16" else coeffs)) <= TC_TOL
    assert o.rel_l2(layer.jacobi_coeffs.grad.cpu(), dC_ref) <= TC_TOL
    assert o.rel_l2(xd.grad.cpu(), dx_ref) <= TC_TOL
    with pytest.raises(ValueError, match="math_mode"):
        kan_b200.HermiteKANLayer(3, 2, 4, math_mode="fp32x3")
    with pytest.raises(RuntimeError, match="not supported"):
        ops.family_forward(ops.make_family("hermite"), x.cuda(), ops.pack_coeffs(coeffs.cuda(), "fp32x3"), 48, 300, 6, "fp32x3")
    with pytest.raises(RuntimeError, match="not supported"):
        ops.family_bwd_dx(ops.make_family("hermite"), x.cuda(), dy.cuda(), coeffs.cuda(), "fp32x3")


def test_chebyshev_through_the_table_equals_the_chebyshev_kernels():
    """Family kind 'chebyshev' drives the table-based kernels with A = 2, C = 1: same values as the layer's own
    kernels up to the different rounding of (2u) P - Q against (2 u) P - 1 Q."""
    g = torch.Generator().manual_seed(3)
    x = torch.randn(3000, 40, generator=g).cuda()
    dy = torch.randn(3000, 24, generator=g).cuda()
    coeffs = (torch.randn(40, 24, 9, generator=g) / 360).cuda()
    fam = ops.make_family("chebyshev")
    packed = ops.pack_coeffs(coeffs, "fp32")
    assert o.rel_l2(ops.family_forward(fam, x, packed, 40, 24, 8), ops.forward(x, packed, 40, 24, 8, "fp32")) <= 1e-6
    assert o.rel_l2(ops.family_bwd_dcoeff(fam, x, dy, 40, 24, 8), ops.bwd_dcoeff(x, dy, 40, 24, 8, "fp32")) <= 1e-6
    assert o.rel_l2(ops.family_bwd_dx(fam, x, dy, coeffs), ops.bwd_dx(x, dy, coeffs, "fp32")) <= 1e-6


def test_dcoeff_accumulates_and_empty_batch():
    fam = ops.make_family("jacobi", alpha=0.5, beta=0.5)
    g = torch.Generator().manual_seed(1)
    x = torch.randn(500, 6, generator=g).cuda()
    dy = torch.randn(500, 4, generator=g).cuda()
    base = torch.full((6, 4, 5), 2.0, device="cuda")
    once = ops.family_bwd_dcoeff(fam, x, dy, 6, 4, 4)
    acc = ops.family_bwd_dcoeff(fam, x, dy, 6, 4, 4, out=base.clone(), accumulate=True)
    assert o.rel_l2(acc, once + 2.0) <= 1e-6
    empty = torch.empty(0, 6, device="cuda")
    assert ops.family_forward(fam, empty, ops.pack_coeffs(base, "fp32"), 6, 4, 4).shape == (0, 4)
    assert not bool(ops.family_bwd_dcoeff(fam, empty, torch.empty(0, 4, device="cuda"), 6, 4, 4).any())


@pytest.mark.parametrize("kind,kw", [("jacobi", {"alpha": 0.5, "beta": -0.3}), ("jacobi", {}),
                                     ("hermite", {}), ("hermite", {"scaling": "probabilist"}),
                                     ("hermite", {"domain": (-2.0, 5.0)}),
                                     ("hermite", {"domain": (-2.0, 5.0), "normalize_domain": False})])
def test_layer_classes_are_drop_ins(kind, kw):
    Layer = kan_b200.JacobiKANLayer if kind == "jacobi" else kan_b200.HermiteKANLayer
    pname = "jacobi_coeffs" if kind == "jacobi" else "hermite_coeffs"
    torch.manual_seed(21)
    layer = Layer(10, 7, 6, **kw)
    torch.manual_seed(21)
    coeffs = po.init_coeffs(10, 7, 6)
    assert torch.equal(getattr(layer, pname).detach(), coeffs)            # same RNG consumption as the reference
    assert list(layer.state_dict()) == [pname]
    assert layer.get_coefficients() is getattr(layer, pname)
    form = layer.get_analytical_form()
    assert form["type"] == Layer.__name__ and form["coefficients"].shape == (10, 7, 7)
    assert form["basis"] == (f"Jacobi-6-{kw.get('alpha', 0.0)}-{kw.get('beta', 0.0)}" if kind == "jacobi"
                             else f"Hermite-6-{kw.get('scaling', 'physicist')}")
    assert "degree=6" in repr(layer)
    with pytest.raises(RuntimeError, match="CUDA"):
        layer(torch.randn(4, 10))
    layer = layer.cuda()
    x = torch.randn(3, 11, 10)
    xd = x.cuda().requires_grad_(True)
    y = layer(xd)                                                          # leading dimensions are flattened
    assert y.shape == (33, 7)
    dy = torch.randn(33, 7)
    y.backward(dy.cuda())
    y_ref, dC_ref, dx_ref = po.forward_backward(dict(kw, kind=kind), x.view(-1, 10), coeffs, dy)
    assert o.rel_l2(y.detach().cpu(), y_ref) <= FP32_TOL
    assert o.rel_l2(getattr(layer, pname).grad.cpu(), dC_ref) <= FP32_TOL
    assert o.rel_l2(xd.grad.cpu().view(-1, 10), dx_ref) <= FP32_TOL
    # the packed copy follows in-place updates of the parameter, and a deep copy is independent
    clone = copy.deepcopy(layer)
    with torch.no_grad():
        getattr(layer, pname).mul_(2.0)
    assert o.rel_l2(layer(xd).detach().cpu(), 2 * y_ref) <= FP32_TOL
    assert o.rel_l2(clone(xd).detach().cpu(), y_ref) <= FP32_TOL
    # the basis object's own methods
    basis = layer.basis_function
    u = basis.normalize_input(x.cuda())
    u_ref = torch.tanh(x) if kind == "jacobi" else po.hermite_normalize(x, kw.get("domain"), kw.get("normalize_domain", True))
    assert o.rel_l2(u.cpu(), u_ref) <= 1e-6
    phi = basis.basis_functions(u)
    phi_ref = (po.jacobi_basis(u_ref, 6, kw.get("alpha", 0.0), kw.get("beta", 0.0)) if kind == "jacobi"
               else po.hermite_basis(u_ref, 6, kw.get("scaling", "physicist")))
    assert phi.shape == (3, 11, 10, 7)
    assert o.rel_l2(phi.cpu(), phi_ref) <= FP32_TOL
    assert o.rel_l2(basis.forward(x.cuda(), getattr(clone, pname).detach()).cpu(), y_ref) <= FP32_TOL


def test_constructor_errors_match_the_reference():
    with pytest.raises(ValueError, match="α, β > -1"):
        kan_b200.JacobiKANLayer(3, 2, 4, alpha=-1.0)
    with pytest.raises(ValueError, match="Invalid scaling"):
        kan_b200.HermiteKANLayer(3, 2, 4, scaling="quantum")


@pytest.mark.parametrize("kind,kw", [("jacobi", {"alpha": 0.0, "beta": 0.0}), ("hermite", {"scaling": "probabilist"})])
def test_short_training_run_follows_the_oracle(kind, kw):
    """Two-layer model, Adam, 20 steps on sin(2 pi x): losses and final coefficients against the same loop on the oracle."""
    Layer = kan_b200.JacobiKANLayer if kind == "jacobi" else kan_b200.HermiteKANLayer
    pname = "jacobi_coeffs" if kind == "jacobi" else "hermite_coeffs"
    fam = dict(kw, kind=kind)
    torch.manual_seed(8)
    ours = torch.nn.Sequential(Layer(1, 8, 5, **kw), Layer(8, 1, 5, **kw))
    ref_params = [getattr(m, pname).detach().clone().requires_grad_(True) for m in ours]
    ours = ours.cuda()
    x = torch.linspace(-1, 1, 128).view(-1, 1)
    t = torch.sin(2 * torch.pi * x)
    opt = kan_b200.optim.Adam(ours.parameters(), lr=0.01)
    ref_opt = torch.optim.Adam(ref_params, lr=0.01)
    xd, td = x.cuda(), t.cuda()
    for step in range(20):
        opt.zero_grad()
        loss = kan_b200.mse_loss(ours(xd), td)
        loss.backward()
        opt.step()
        ref_opt.zero_grad()
        ref_loss = torch.nn.functional.mse_loss(po.forward(fam, po.forward(fam, x, ref_params[0]), ref_params[1]), t)
        ref_loss.backward()
        ref_opt.step()
        assert abs(float(loss) - float(ref_loss)) <= 1e-3 * abs(float(ref_loss))
    for m, p in zip(ours, ref_params):
        assert o.rel_l2(getattr(m, pname).detach().cpu(), p.detach()) <= 5e-3
