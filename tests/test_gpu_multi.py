"""Data-parallel checks over NCCL on every GPU of the box (skipped on a single-GPU box): sharded inference
reproduces the single-GPU rows bit for bit, the all-reduced coefficient gradient matches the full-batch
gradient, one sharded training step leaves identical coefficients on every rank (also when the step, collective
included, is replayed as a CUDA graph), and a layer sharded over its output columns gives the unsharded layer's y,
dC and dx."""
import datetime
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    # a short collective timeout: a rank that failed before a collective ends the others' wait with an error
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank),
                            timeout=datetime.timedelta(seconds=120))
    try:
        import kan_b200
        from kan_b200 import dp, ops
        from oracle import chebykan_oracle as o
        ok = True
        # --- fp32: gradient of the full batch = sum of the shards' gradients
        torch.manual_seed(0)
        layer = kan_b200.ChebyKANLayer(64, 48, 8).cuda()
        g = torch.Generator().manual_seed(1)
        B = 4096 + 8                                    # not a multiple of the world size: shards differ by one row
        x = torch.randn(B, 64, generator=g)
        dy = torch.randn(B, 48, generator=g)
        b, e = dp.shard_rows(B, rank, world)
        buf = dp.FlatGradBuffer(layer.parameters())
        y = layer(x[b:e].cuda())
        y.backward(dy[b:e].cuda())
        buf.all_reduce()
        torch.cuda.synchronize()
        y_ref, dC_ref, _ = o.forward_backward(x, layer.cheby_coeffs.detach().cpu(), dy, need_dx=False)
        ok = ok and o.rel_l2(y.detach().cpu(), y_ref[b:e]) <= 1e-5
        ok = ok and o.rel_l2(layer.cheby_coeffs.grad.cpu(), dC_ref) <= 1e-5
        # --- tensor-core forward: the shards' rows, concatenated, equal the single-GPU result bit for bit, on narrow
        # and on wide layers (a row's value does not depend on which tile or which GPU computes it)
        for mode in ("bf16", "tf32"):
            for n_in, n_out, exact in ((64, 64, True), (256, 640, True)):
                torch.manual_seed(2)
                layer_w = kan_b200.ChebyKANLayer(n_in, n_out, 4, math_mode=mode).cuda()
                Bw = 2048 * world
                xw = torch.randn(Bw, n_in, generator=torch.Generator().manual_seed(3)).cuda()
                with torch.no_grad():
                    full = layer_w(xw)
                    mine = layer_w(xw[rank * 2048:(rank + 1) * 2048].contiguous())
                parts = [torch.empty_like(mine) for _ in range(world)]
                dist.all_gather(parts, mine)
                cat = torch.cat(parts)
                ok = ok and (torch.equal(cat, full) if exact else o.rel_l2(cat, full) <= 1e-5)
        # --- one sharded SGD step (tf32): every rank ends with the same coefficients, equal to the oracle's step
        torch.manual_seed(5)
        model = kan_b200.ChebyKANLayer(32, 16, 6, math_mode="tf32").cuda()
        start = model.cheby_coeffs.detach().cpu().clone()
        Bt = 1024 * world
        gt = torch.Generator().manual_seed(7)
        xt, tt = torch.randn(Bt, 32, generator=gt), torch.randn(Bt, 16, generator=gt)
        bt, et = dp.shard_rows(Bt, rank, world)
        gbuf = dp.FlatGradBuffer(model.parameters())
        opt = kan_b200.optim.SGD(list(model.parameters()), lr=0.5)
        gbuf.zero()
        loss = kan_b200.mse_loss(model(xt[bt:et].cuda()), tt[bt:et].cuda(), n_mean=Bt * 16)
        loss.backward()
        gbuf.all_reduce()
        opt.step()
        ops.check_status()
        mine = model.cheby_coeffs.detach()
        allw = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(allw, mine)
        ok = ok and all(torch.equal(allw[0], w) for w in allw)
        cr = start.clone().requires_grad_(True)
        torch.nn.functional.mse_loss(o.forward(xt, cr), tt).backward()
        expect = start - 0.5 * cr.grad
        ok = ok and o.rel_l2(mine.cpu() - start, expect - start) <= 2e-3
        # --- the same kind of step replayed as one CUDA graph per rank, all-reduce inside the graph: three replays
        # leave the coefficients that the eager data-parallel loop leaves, identical on every rank
        torch.manual_seed(9)
        mk = lambda: torch.nn.Sequential(kan_b200.ChebyKANLayer(64, 64, 8, math_mode="tf32"),
                                         kan_b200.ChebyKANLayer(64, 32, 8, math_mode="tf32")).cuda()
        m_e, m_g = mk(), mk()
        m_g.load_state_dict(m_e.state_dict())
        Bg = 2048 * world
        gg = torch.Generator().manual_seed(13)
        xg_, tg_ = torch.randn(Bg, 64, generator=gg), torch.randn(Bg, 32, generator=gg)
        bg, eg = dp.shard_rows(Bg, rank, world)
        xs, ts = xg_[bg:eg].cuda(), tg_[bg:eg].cuda()
        loss_fn = lambda y_, t_: kan_b200.mse_loss(y_, t_, n_mean=Bg * 32)
        gstep = kan_b200.graph.GraphedTrainStep(m_g, loss_fn, kan_b200.optim.SGD(list(m_g.parameters()), lr=0.1), xs, ts)
        for _ in range(3):
            gstep()
        ebuf = dp.FlatGradBuffer(m_e.parameters())
        eopt = kan_b200.optim.SGD(list(m_e.parameters()), lr=0.1)
        for _ in range(3 + 3):                          # the graphed step ran three eager warm-up steps first
            ebuf.zero()
            loss_fn(m_e(xs), ts).backward()
            ebuf.all_reduce()
            eopt.step()
        torch.cuda.synchronize()
        ops.check_status()
        gstep.close()                                   # destroy_process_group waits for graphs that hold a collective
        with pytest.raises(RuntimeError):
            gstep()
        for pe, pg in zip(m_e.parameters(), m_g.parameters()):
            ok = ok and o.rel_l2(pg.detach().cpu(), pe.detach().cpu()) <= 1e-6
            allg = [torch.empty_like(pg.detach()) for _ in range(world)]
            dist.all_gather(allg, pg.detach().contiguous())
            ok = ok and all(torch.equal(allg[0], w) for w in allg)
        # --- the output dimension as a second sharding axis: every rank holds a block of output columns of one layer
        # (Chebyshev fp32 and a Jacobi layer), sees all rows, and dx is summed over the ranks
        from oracle import polykan_oracle as po
        n_out = 8 * world + 3                           # shards differ by one column
        go = torch.Generator().manual_seed(11)
        xo, dyo = torch.randn(333, 40, generator=go), torch.randn(333, n_out, generator=go)
        full = torch.randn(40, n_out, 6, generator=go) / 240
        cases = ((lambda n: kan_b200.ChebyKANLayer(40, n, 5), lambda x, c: o.forward(x, c)),
                 (lambda n: kan_b200.JacobiKANLayer(40, n, 5, alpha=0.5, beta=0.25),
                  lambda x, c: po.jacobi_forward(x, c, 0.5, 0.25)))
        for make, ref_fwd in cases:
            tp = dp.OutputParallel(lambda n: make(n).cuda(), n_out, full_coefficients=full.cuda(), gather_output=True)
            xg = xo.cuda().requires_grad_(True)
            yo = tp(xg)
            yo.backward(dyo.cuda())
            xr, cr = xo.clone().requires_grad_(True), full.clone().requires_grad_(True)
            y_ref = ref_fwd(xr, cr)
            y_ref.backward(dyo)
            ok = ok and o.rel_l2(yo.detach().cpu(), y_ref.detach()) <= 1e-5
            ok = ok and o.rel_l2(xg.grad.cpu(), xr.grad) <= 1e-5
            ok = ok and o.rel_l2(tp.shard.get_coefficients().grad.cpu(), cr.grad[:, tp.begin:tp.end]) <= 1e-5
            ok = ok and torch.equal(tp.full_coefficients().cpu(), full)
        results[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least two GPUs")
def test_data_parallel_on_all_gpus():
    world = min(torch.cuda.device_count(), 8)
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        results = mgr.dict()
        port = 29600 + os.getpid() % 2000
        procs = [ctx.Process(target=_worker, args=(r, world, port, results)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(timeout=600)
        stuck = [p for p in procs if p.exitcode is None]
        for p in stuck:                                  # never leave a child behind on the GPU
            p.terminate()
            p.join(timeout=30)
        assert not stuck
        assert all(p.exitcode == 0 for p in procs)
        assert dict(results) == {r: True for r in range(world)}
