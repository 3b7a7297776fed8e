"""CPU tests of the Jacobi / Hermite oracle: against the unmodified reference (when its tree is present), against
the committed golden vectors and known polynomial values; and of the library's host-side recurrence table."""
import numpy as np
import pytest
import torch

from oracle import chebykan_oracle as o
from oracle import polykan_oracle as po
from oracle import ref_loader

CASE_NAMES = ["legendre_d6", "jacobi_a05_bm03_d9", "jacobi_a2_b1_d16", "jacobi_cheb1_d8", "jacobi_d0", "jacobi_d1",
              "jacobi_wide_out", "hermite_phys_d6", "hermite_prob_d9", "hermite_phys_d12_uniform",
              "hermite_domain_affine", "hermite_domain_no_normalize", "hermite_d0", "hermite_d1"]


def test_golden_file_holds_exactly_these_cases(golden_poly):
    assert sorted(golden_poly) == sorted(CASE_NAMES)


@pytest.mark.parametrize("name", CASE_NAMES)
def test_oracle_matches_golden(golden_poly, name):
    c = golden_poly[name]
    y, dC, dx = po.forward_backward(c["family"], torch.from_numpy(c["x"]), torch.from_numpy(c["coeffs"]),
                                    torch.from_numpy(c["dy"]))
    # bit-exact on the machine that generated the fixtures; other CPUs may pick other vector kernels
    assert o.rel_l2(y, c["y"]) <= 2e-6
    assert o.rel_l2(dC, c["dC"]) <= 2e-6
    if np.any(c["dx"]):
        assert o.rel_l2(dx, c["dx"]) <= 2e-6
    else:
        assert not bool(dx.any())


@pytest.mark.skipif(not ref_loader.available(), reason="reference tree not on this machine")
@pytest.mark.parametrize("kind,kw,rows,n_in,n_out,deg", [
    ("jacobi", {}, 50, 8, 6, 8), ("jacobi", {"alpha": 0.5, "beta": -0.3}, 33, 7, 5, 9),
    ("jacobi", {"alpha": 1.5, "beta": 2.0}, 21, 5, 4, 32), ("jacobi", {}, 10, 3, 2, 0),
    ("hermite", {}, 50, 8, 6, 8), ("hermite", {"scaling": "probabilist"}, 33, 7, 5, 9),
    ("hermite", {"domain": (-2.0, 5.0)}, 21, 5, 4, 5), ("hermite", {"domain": (-2.0, 5.0), "normalize_domain": False}, 21, 5, 4, 5),
    ("hermite", {"domain": (-float("inf"), 4.0)}, 21, 5, 4, 3), ("hermite", {"scaling": "probabilist"}, 10, 3, 2, 0),
])
def test_oracle_bit_exact_vs_reference(kind, kw, rows, n_in, n_out, deg):
    ref_loader.load()
    from kan.layers.hermitekan import HermiteKANLayer
    from kan.layers.jacobikan import JacobiKANLayer
    torch.manual_seed(13)
    layer = (JacobiKANLayer if kind == "jacobi" else HermiteKANLayer)(n_in, n_out, deg, **kw)
    torch.manual_seed(13)
    coeffs = po.init_coeffs(n_in, n_out, deg)
    assert torch.equal(layer.get_coefficients().detach(), coeffs)     # same RNG consumption
    x = torch.randn(rows, n_in, requires_grad=True)
    y = layer(x)
    dy = torch.randn_like(y)
    y.backward(dy)
    y2, dC2, dx2 = po.forward_backward(dict(kw, kind=kind), x.detach(), coeffs, dy)
    assert torch.equal(y.detach(), y2)
    assert torch.equal(layer.get_coefficients().grad, dC2)
    assert torch.equal(x.grad if x.grad is not None else torch.zeros_like(x), dx2)


def test_known_polynomial_values():
    u = torch.tensor([-1.0, -0.5, 0.0, 0.25, 1.0], dtype=torch.float64)
    leg = po.jacobi_basis(u, 4)                      # alpha = beta = 0: Legendre
    assert torch.allclose(leg[:, 2], (3 * u ** 2 - 1) / 2)
    assert torch.allclose(leg[:, 3], (5 * u ** 3 - 3 * u) / 2)
    assert torch.allclose(leg[:, 4], (35 * u ** 4 - 30 * u ** 2 + 3) / 8)
    # alpha = beta = -1/2: Chebyshev of the first kind up to the factor binom(n - 1/2, n)
    jac = po.jacobi_basis(u, 3, -0.5, -0.5)
    cheb = o.basis_recurrence(u.view(1, -1), 3)[0]
    assert torch.allclose(jac[:, 2], cheb[:, 2] * 3 / 8) and torch.allclose(jac[:, 3], cheb[:, 3] * 5 / 16)
    # P_n^(a,b)(1) = binom(n + a, n)
    assert torch.allclose(po.jacobi_basis(torch.ones(1, dtype=torch.float64), 3, 2.0, 1.0)[0],
                          torch.tensor([1.0, 3.0, 6.0, 10.0], dtype=torch.float64))
    h = po.hermite_basis(u, 4)
    assert torch.allclose(h[:, 3], 8 * u ** 3 - 12 * u) and torch.allclose(h[:, 4], 16 * u ** 4 - 48 * u ** 2 + 12)
    he = po.hermite_basis(u, 4, "probabilist")
    assert torch.allclose(he[:, 3], u ** 3 - 3 * u) and torch.allclose(he[:, 4], u ** 4 - 6 * u ** 2 + 3)
    x = torch.tensor([[-7.0, 0.0, 7.0]])
    assert torch.allclose(po.hermite_normalize(x), torch.tensor([[-3.0, 0.0, 3.0]]), atol=1e-5)
    assert torch.equal(po.hermite_normalize(torch.tensor([-2.0, 1.5, 5.0]), (-2.0, 5.0)), torch.tensor([-3.0, 0.0, 3.0]))


@pytest.mark.parametrize("kind,kw,okw", [
    ("jacobi", {}, {"kind": "jacobi"}),
    ("jacobi", {"alpha": 0.5, "beta": -0.3}, {"kind": "jacobi", "alpha": 0.5, "beta": -0.3}),
    ("jacobi", {"alpha": 2.0, "beta": 1.0}, {"kind": "jacobi", "alpha": 2.0, "beta": 1.0}),
    ("hermite", {}, {"kind": "hermite"}),
    ("hermite_prob", {}, {"kind": "hermite", "scaling": "probabilist"}),
    ("chebyshev", {}, None),
])
def test_library_recurrence_table_reproduces_the_basis(built_lib, kind, kw, okw):
    """The table the kernels take as a launch parameter (host code, needs no GPU), evaluated in float64, gives the
    oracle's polynomials up to the fp32 rounding of its entries."""
    from kan_b200 import ops
    deg = 24
    a, b, c = [t.double() for t in ops.family_table(ops.make_family(kind, **kw), deg)]
    u = torch.linspace(-1, 1, 101, dtype=torch.float64) * (3 if kind.startswith("hermite") else 1)
    cols = [torch.ones_like(u), a[1] * u + b[1]]
    assert float(c[1]) == 0.0
    for d in range(2, deg + 1):
        cols.append((a[d] * u + b[d]) * cols[-1] - c[d] * cols[-2])
    phi = torch.stack(cols, -1)
    if okw is None:
        ref = o.basis_recurrence(u.view(1, -1), deg)[0]
    elif okw["kind"] == "jacobi":
        ref = po.jacobi_basis(u, deg, okw.get("alpha", 0.0), okw.get("beta", 0.0))
    else:
        ref = po.hermite_basis(u, deg, okw.get("scaling", "physicist"))
    for d in range(deg + 1):
        assert float((phi[:, d] - ref[:, d]).abs().max()) <= 1e-5 * float(ref[:, d].abs().max())


def test_library_rejects_bad_families(built_lib):
    from kan_b200 import _lib, ops
    with pytest.raises(ValueError):
        ops.make_family("laguerre")
    for fam in (ops.make_family("jacobi", alpha=-1.0), ops.make_family("jacobi", beta=-2.0),
                ops.make_family("jacobi", alpha=float("nan")), _lib.Family(9, 0, 0, 0, 0, 0, 0),
                ops.make_family("hermite", scale=float("inf"))):
        with pytest.raises(RuntimeError, match="invalid argument"):
            ops.family_table(fam, 4)
    with pytest.raises(RuntimeError, match="invalid argument"):
        ops.family_table(ops.make_family("jacobi"), 128)
