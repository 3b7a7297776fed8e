"""Data-parallel checks over NCCL on every GPU of the box (skipped on a single-GPU box): sharded inference
reproduces the single-GPU rows bit for bit, the all-reduced coefficient gradient matches the full-batch
gradient, one sharded training step leaves identical coefficients on every rank, and a layer sharded over its
output columns gives the unsharded layer's y, dC and dx."""
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
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
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
            assert p.exitcode == 0
        assert dict(results) == {r: True for r in range(world)}
