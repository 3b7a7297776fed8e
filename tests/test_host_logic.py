"""CPU tests of the host-side mirror of the reference interface and of the
data-parallel plumbing (gloo, world size 2)."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import kan_b200
from kan_b200 import dp, workloads
from oracle import chebykan_oracle as o
from oracle import ref_loader


def test_constructor_draws_reference_weights():
    torch.manual_seed(123)
    layer = kan_b200.ChebyKANLayer(12, 7, 5)
    torch.manual_seed(123)
    assert torch.equal(layer.cheby_coeffs.detach(), o.init_coeffs(12, 7, 5))
    assert layer.cheby_coeffs.shape == (12, 7, 6) and layer.cheby_coeffs.dtype == torch.float32
    torch.manual_seed(123)
    scaled = kan_b200.ChebyKANLayer(12, 7, 5, init_scale=0.5)
    assert abs(float(scaled.cheby_coeffs.detach().std()) - 0.5) < 0.05


def test_module_surface_matches_reference():
    layer = kan_b200.ChebyKANLayer(64, 64, 8)
    assert list(layer.state_dict().keys()) == ["cheby_coeffs"]
    assert [n for n, _ in layer.named_parameters()] == ["cheby_coeffs"]
    assert list(layer.named_buffers()) == []
    assert repr(layer) == "ChebyKANLayer(input_dim=64, output_dim=64, degree=8)"
    assert layer.get_coefficients() is layer.cheby_coeffs
    form = layer.get_analytical_form()
    assert set(form) == {"type", "input_dim", "output_dim", "degree", "basis", "coefficients"}
    assert form["type"] == "ChebyKANLayer" and form["basis"] == "Chebyshev-8"
    assert form["coefficients"].shape == (64, 64, 9)
    assert layer.basis is layer.basis_function and layer.basis.name == "Chebyshev-8"
    assert layer.basis.domain == (-1, 1) and layer.input_dim == 64 and layer.output_dim == 64
    assert isinstance(layer, kan_b200.KANLayer)
    with pytest.raises(ValueError):
        kan_b200.ChebyKANLayer(4, 4, 2, math_mode="fp16")


def test_no_cpu_fallback():
    layer = kan_b200.ChebyKANLayer(4, 3, 2)
    with pytest.raises(RuntimeError, match="CUDA"):
        layer(torch.randn(5, 4))
    with pytest.raises(RuntimeError):
        layer(torch.randn(5, 3))          # wrong last dimension: view fails like the reference


def test_product_never_imports_the_oracle():
    root = os.path.dirname(os.path.abspath(kan_b200.__file__))
    for dirpath, _, files in os.walk(root):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text.replace("oracle/", "").lower() or f == "never", f


@pytest.mark.skipif(not ref_loader.available(), reason="reference tree not on this machine")
def test_install_into_reference_registry():
    kan = ref_loader.load()
    from kan.layers.chebykan import ChebyKANLayer as RefLayer
    saved = (kan.layers.LAYER_REGISTRY['chebykan'], kan.layers.ChebyKANLayer, kan.ChebyKANLayer)
    try:
        cls = kan_b200.install_into_reference()
        layer = kan.layers.get_layer('chebykan', input_dim=5, output_dim=3, degree=4)
        assert isinstance(layer, cls)
        assert isinstance(layer, kan.layers.base.KANLayer)
        assert isinstance(layer.basis_function, kan.basis.chebyshev.ChebyshevBasis)
        # checkpoints move both ways
        torch.manual_seed(9)
        ref = RefLayer(5, 3, 4)
        layer.load_state_dict(ref.state_dict())
        assert torch.equal(layer.cheby_coeffs, ref.cheby_coeffs)
        ref.load_state_dict(layer.state_dict())
        # the reference's symbolic export dispatches on the basis object and reads the
        # coefficients; it must treat the drop-in exactly as it treats its own layer
        # (in reference version 0.4.0 that is the same AttributeError for both)
        from kan.utils.symbolic import get_layer_symbolic_expr

        def outcome(l):
            try:
                return ("ok", len(get_layer_symbolic_expr(l)))
            except Exception as e:  # noqa: BLE001
                return (type(e).__name__, str(e))
        assert outcome(layer) == outcome(ref)
        seq = kan.layers.base.KANSequential(layer)
        forms = seq.get_analytical_form()          # isinstance(module, KANLayer) dispatch
        assert len(forms) == 1 and forms[0]['type'] == 'ChebyKANLayer'
    finally:
        kan.layers.LAYER_REGISTRY['chebykan'], kan.layers.ChebyKANLayer, kan.ChebyKANLayer = saved


def test_shard_rows_partition():
    assert dp.world_info_of(None) == (0, 1)              # no process group in this process
    for n, w in [(65536, 8), (100, 3), (7, 8), (0, 2)]:
        spans = [dp.shard_rows(n, r, w) for r in range(w)]
        assert spans[0][0] == 0 and spans[-1][1] == n
        for a, b in zip(spans, spans[1:]):
            assert a[1] == b[0]
        sizes = [e - b for b, e in spans]
        assert max(sizes) - min(sizes) <= 1


def test_workload_generators():
    for name, cfg in workloads.CONFIGS.items():
        x, tgt = workloads.make_inputs(cfg, batch=64 if name != "cfg1" else None)
        assert x.dtype == torch.float32 and x.shape[1] == cfg.layers[0][0]
        x2, _ = workloads.make_inputs(cfg, batch=64 if name != "cfg1" else None)
        assert torch.equal(x, x2)
    x, labels = workloads.make_inputs(workloads.CONFIGS["cfg2"], batch=256)
    frac_zero = float((x == 0).float().mean())
    assert 0.75 < frac_zero < 0.85 and labels.min() >= 0 and labels.max() <= 9
    assert workloads.flops_per_sample(workloads.CONFIGS["cfg3"]) == 18874368
    m = workloads.build_model(workloads.CONFIGS["cfg4"], kan_b200.ChebyKANLayer)
    assert len(m) == 7 and isinstance(m[1], torch.nn.LayerNorm)


def _dp_worker(rank, world, port, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # every rank owns a block of rows; the gradient of a sum over rows is the sum of the blocks'
        torch.manual_seed(0)
        coeffs = o.init_coeffs(6, 4, 3)
        g = torch.Generator().manual_seed(1)
        x = torch.randn(40, 6, generator=g)
        dy = torch.randn(40, 4, generator=g)
        b, e = dp.shard_rows(40, rank, world)
        _, dC_local, _ = o.forward_backward(x[b:e], coeffs, dy[b:e], need_dx=False)
        p1 = torch.nn.Parameter(coeffs.clone())
        p2 = torch.nn.Parameter(torch.zeros(5))
        buf = dp.FlatGradBuffer([p1, p2])
        assert p1.grad.data_ptr() == buf.flat.data_ptr()
        p1.grad.copy_(dC_local)
        p2.grad.fill_(float(rank + 1))
        buf.all_reduce()
        _, dC_full, _ = o.forward_backward(x, coeffs, dy, need_dx=False)
        ok = o.rel_l2(p1.grad, dC_full) < 1e-6 and torch.allclose(p2.grad, torch.full((5,), 3.0))
        assert dp.world_info() == (rank, world)
        assert dp.world_info_of(None) == (rank, world)
        # zero_grad(set_to_none=True) drops the aliases; backward then installs fresh tensors: the next
        # all_reduce must still cover them
        p1.grad = None
        p2.grad = None
        p1.grad = dC_local.clone()
        p2.grad = torch.full((5,), float(rank + 1))
        buf.all_reduce()
        ok = ok and o.rel_l2(p1.grad, dC_full) < 1e-6 and torch.allclose(p2.grad, torch.full((5,), 3.0))
        ok = ok and p1.grad.data_ptr() == buf.flat.data_ptr()
        results[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_flat_grad_allreduce_gloo_world2():
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        results = mgr.dict()
        port = 29500 + os.getpid() % 2000
        procs = [ctx.Process(target=_dp_worker, args=(r, 2, port, results)) for r in range(2)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(timeout=180)
            assert p.exitcode == 0
        assert dict(results) == {0: True, 1: True}


def _tp_worker(rank, world, port, results):
    """Output-sharded layer on `world` CPU ranks (the oracle layer stands in for the CUDA layer: the sharding logic
    does not depend on which layer class computes): y, dC and dx equal the unsharded layer's."""
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from _util import OracleLayer

        class Layer(OracleLayer):
            def get_coefficients(self):
                return self.cheby_coeffs

        torch.manual_seed(3)
        full = o.init_coeffs(6, 7, 3)                      # 7 outputs over 2 ranks: shards of 4 and 3 columns
        g = torch.Generator().manual_seed(4)
        x = torch.randn(20, 6, generator=g)
        dy = torch.randn(20, 7, generator=g)
        y_ref, dC_ref, dx_ref = o.forward_backward(x, full, dy)
        ok = True
        for gather in (False, True):
            tp = dp.OutputParallel(lambda n: Layer(6, n, 3), 7, full_coefficients=full, gather_output=gather)
            xr = x.clone().requires_grad_(True)
            y = tp(xr)
            b, e = dp.shard_outputs(7, rank, world)
            if gather:
                ok = ok and y.shape == (20, 7) and torch.equal(y.detach(), y_ref)
                y.backward(dy)
            else:
                ok = ok and y.shape == (20, e - b) and torch.equal(y.detach(), y_ref[:, b:e])
                y.backward(dy[:, b:e])
            ok = ok and o.rel_l2(tp.shard.cheby_coeffs.grad, dC_ref[:, b:e]) < 1e-6
            ok = ok and o.rel_l2(xr.grad, dx_ref) < 1e-6         # summed over the ranks' column blocks
            ok = ok and torch.equal(tp.full_coefficients(), full)
        results[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_output_parallel_gloo_world2():
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        results = mgr.dict()
        port = 31500 + os.getpid() % 2000
        procs = [ctx.Process(target=_tp_worker, args=(r, 2, port, results)) for r in range(2)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(timeout=180)
            assert p.exitcode == 0
        assert dict(results) == {0: True, 1: True}


def test_output_parallel_single_process_is_the_plain_layer():
    assert dp.shard_outputs(7, 0, 2) == (0, 4) and dp.shard_outputs(7, 1, 2) == (4, 7)
    tp = dp.OutputParallel(lambda n: kan_b200.ChebyKANLayer(5, n, 2), 9)
    assert (tp.world, tp.begin, tp.end) == (1, 0, 9) and tp.shard.cheby_coeffs.shape == (5, 9, 3)
    with pytest.raises(ValueError):
        dp.OutputParallel(lambda n: kan_b200.ChebyKANLayer(5, max(n, 1), 2), 0)


def test_ref_loader_search_order(tmp_path, monkeypatch):
    """$KAN_REF first, then baseline/_ref/ under the repository, then the container's read-only mount."""
    fake = tmp_path / "ref"
    (fake / "kan" / "layers").mkdir(parents=True)
    (fake / "kan" / "layers" / "chebykan.py").write_text("# marker\n")
    monkeypatch.setenv("KAN_REF", str(fake))
    cands = ref_loader.candidate_roots()
    assert cands[0] == str(fake)
    assert cands[1].endswith(os.path.join("baseline", "_ref")) and cands[2] == ref_loader.DEFAULT_MOUNT
    assert ref_loader.reference_root() == str(fake)
    monkeypatch.setenv("KAN_REF", str(tmp_path / "missing"))
    assert ref_loader.reference_root() in (None, cands[1], cands[2])


def test_status_word_raises_and_clears(monkeypatch):
    """A non-zero status word (a bounded device-side wait that gave up) becomes a RuntimeError at the next check."""
    from kan_b200 import ops
    word = torch.tensor([3], dtype=torch.int32)          # a CPU stand-in for the device word
    monkeypatch.setattr(ops, "_status", {0: word})
    with pytest.raises(RuntimeError, match="role code 3"):
        ops.check_status()
    assert int(word) == 0                                  # cleared, so that the next check starts clean
    ops.check_status()                                     # nothing pending: no error


def test_flat_grad_buffer_survives_zero_grad_set_to_none():
    """zero_grad(set_to_none=True) drops p.grad; the buffer re-attaches its views, keeping what backward produced."""
    p1 = torch.nn.Parameter(torch.randn(3, 5))
    p2 = torch.nn.Parameter(torch.randn(7))
    buf = dp.FlatGradBuffer([p1, p2])
    torch.optim.SGD([p1, p2], lr=0.1).zero_grad()          # torch's default: set_to_none=True
    assert p1.grad is None and p2.grad is None
    (p1.sum() * 2 + p2.sum() * 3).backward()               # installs fresh tensors that do not alias the buffer
    assert p1.grad.data_ptr() != buf.flat.data_ptr()
    buf.all_reduce()                                       # single process: no collective, but the views are re-attached
    assert p1.grad.data_ptr() == buf.flat.data_ptr()
    assert torch.equal(buf.flat[:15], torch.full((15,), 2.0)) and torch.equal(p2.grad, torch.full((7,), 3.0))
    buf.zero()
    assert float(buf.flat.abs().sum()) == 0.0 and p2.grad.data_ptr() == buf.flat[16:].data_ptr()
