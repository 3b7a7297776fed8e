"""Two-GPU data-parallel checks over NCCL (skipped on a single-GPU box):
sharded inference reproduces the single-GPU rows bit for bit, and the
all-reduced coefficient gradient matches the full-batch gradient."""
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
        from kan_b200 import dp
        from oracle import chebykan_oracle as o
        torch.manual_seed(0)
        layer = kan_b200.ChebyKANLayer(64, 48, 8).cuda()
        g = torch.Generator().manual_seed(1)
        x = torch.randn(4096, 64, generator=g)
        dy = torch.randn(4096, 48, generator=g)
        b, e = dp.shard_rows(4096, rank, world)
        buf = dp.FlatGradBuffer(layer.parameters())
        y = layer(x[b:e].cuda())
        y.backward(dy[b:e].cuda())
        buf.all_reduce()
        torch.cuda.synchronize()
        y_ref, dC_ref, _ = o.forward_backward(x, layer.cheby_coeffs.detach().cpu(), dy, need_dx=False)
        ok_y = o.rel_l2(y.detach().cpu(), y_ref[b:e]) <= 1e-5
        ok_g = o.rel_l2(layer.cheby_coeffs.grad.cpu(), dC_ref) <= 1e-5
        results[rank] = bool(ok_y and ok_g)
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_rank_data_parallel():
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        results = mgr.dict()
        port = 29600 + os.getpid() % 2000
        procs = [ctx.Process(target=_worker, args=(r, 2, port, results)) for r in range(2)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(timeout=600)
            assert p.exitcode == 0
        assert dict(results) == {0: True, 1: True}
