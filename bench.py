#!/usr/bin/env python
"""Benchmark of the ChebyKAN layer forward (configuration 3: 65536 x 1024 -> 1024, degree 8).

    python bench.py --gpus N --steps K --warmup W [--mode bf16|tf32|fp32]
    python bench.py --impl reference ...        # the reference's CPU path on the host cores

One "step" is one forward pass of the layer over one batch of synthetic input.
With N > 1 (launched by torch.distributed.run, one rank per GPU) every rank
runs the full configuration-3 batch on its own GPU with replicated
coefficients: rows are independent, so inference has no collective
("weak" scaling; value = rows of all ranks / max-over-ranks time).
Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

METRIC = "chebykan_layer_fwd_samples_per_s"
UNIT = "samples/s"
CFG = dict(workload="cfg3: ChebyKANLayer fwd, batch 65536 per GPU, in=1024, out=1024, degree=8, x~N(0,1) fp32",
           batch_per_gpu=65536, input_dim=1024, output_dim=1024, degree=8)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm_gbs=p["hbm_gbs"], bf16_tflops=p["bf16_tflops"],
                    bf16_tflops_sustained=p.get("bf16_tflops_sustained"), source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed region runs (read-only)."""

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thr = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        names = {
            getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.005)

    def start(self):
        if self.nv is not None:
            self._thr = threading.Thread(target=self._run, daemon=True)
            self._thr.start()

    def stop(self):
        if self._thr is not None:
            self._stop.set()
            self._thr.join()
        med = statistics.median(self.samples) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


def cpu_reference_throughput(rows: int, max_seconds: float, seed: int = 1003):
    """The reference's CPU path for this layer, restated op for op (torch CPU kernels), all host threads."""
    from oracle import chebykan_oracle as o
    torch.set_num_threads(os.cpu_count() or 1)
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(rows, CFG["input_dim"], generator=g)
    torch.manual_seed(seed)
    coeffs = o.init_coeffs(CFG["input_dim"], CFG["output_dim"], CFG["degree"])
    o.forward(x[:256], coeffs)  # warm the thread pool
    best = float("inf")
    times = []
    while sum(times) < max_seconds and len(times) < 50:
        t0 = time.perf_counter()
        o.forward(x, coeffs)
        dt = time.perf_counter() - t0
        times.append(dt)
        best = min(best, dt)
    return rows / best, torch.get_num_threads(), times


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    rows = 4096
    from oracle import chebykan_oracle as o
    torch.set_num_threads(os.cpu_count() or 1)
    g = torch.Generator().manual_seed(1003)
    x = torch.randn(rows, CFG["input_dim"], generator=g)
    torch.manual_seed(1003)
    coeffs = o.init_coeffs(CFG["input_dim"], CFG["output_dim"], CFG["degree"])
    for _ in range(args.warmup):
        o.forward(x, coeffs)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        o.forward(x, coeffs)
    dt = time.perf_counter() - t0
    value = rows * args.steps / dt
    sample = f"{rows} of 65536 rows per step (closed-form basis + einsum, torch CPU fp32)"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": dict(CFG, rows_per_step=rows),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
                         "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


def run_ours(args):
    import torch.distributed as dist
    import kan_b200
    from kan_b200 import ops

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    B, n_in, n_out, deg = CFG["batch_per_gpu"], CFG["input_dim"], CFG["output_dim"], CFG["degree"]
    if args.shape:
        B, n_in, n_out, deg = [int(v) for v in args.shape.split(",")]
    if args.batch:
        B = args.batch
    mode = args.mode
    torch.manual_seed(1003)
    layer = kan_b200.ChebyKANLayer(n_in, n_out, deg, math_mode=mode).to(dev)
    for p in layer.parameters():
        p.requires_grad_(False)
    g = torch.Generator().manual_seed(1003 + rank)
    x_host = torch.randn(B, n_in, generator=g).pin_memory()
    y_host = torch.empty(B, n_out, dtype=torch.float32).pin_memory()
    x = x_host.to(dev)
    packed = ops.pack_coeffs(layer.cheby_coeffs.detach(), mode)
    y = torch.empty(B, n_out, dtype=torch.float32, device=dev)

    if args.op == "fwd":
        def step():
            ops.forward(x, packed, n_in, n_out, deg, mode, out=y)
    else:
        # single backward kernels on the same shape (not the headline metric): dY ~ N(0,1)
        dy = torch.randn(B, n_out, device=dev)
        dc = torch.empty(n_in, n_out, deg + 1, device=dev)
        dx = torch.empty(B, n_in, device=dev)
        cdev = layer.cheby_coeffs.detach()
        if args.op == "dcoeff":
            def step():
                ops.bwd_dcoeff(x, dy, n_in, n_out, deg, mode, out=dc)
        else:
            def step():
                ops.bwd_dx(x, dy, cdev, mode, out=dx)
        args.no_e2e = True

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    sampler = ClockSampler(local) if rank == 0 else None
    if sampler:
        sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    ev0.record()
    for _ in range(args.steps):
        step()
    ev1.record()
    barrier()
    clocks = sampler.stop() if sampler else None
    ops.check_status()
    ms_total = ev0.elapsed_time(ev1)
    t = torch.tensor([ms_total], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_total = float(t.item())
    ms_step = ms_total / args.steps
    value = world * B / (ms_step * 1e-3)

    # end to end through the layer's public call with host buffers: H2D of x, forward, D2H of y
    e2e_steps = max(3, min(args.steps, 10))

    def e2e_step():
        # the layer's public host-buffer call: H2D of x, forward, D2H of y, pipelined in row blocks
        layer.forward_host(x_host, out=y_host)

    e2e_value = None
    if not args.no_e2e:
        e2e_step()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(e2e_steps):
            e2e_step()
        e1.record()
        barrier()
        te = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(te, op=dist.ReduceOp.MAX)
        e2e_value = world * B / (float(te.item()) / e2e_steps * 1e-3)
        ops.check_status()

    if rank == 0:
        peaks = measured_peaks()
        flops = 2.0 * B * n_in * (deg + 1) * n_out
        achieved = flops / (ms_step * 1e-3) / 1e12
        if mode == "fp32":
            peak, peak_note = 148 * 128 * 2 * 1.965e9 / 1e12, "nominal FFMA peak (148 SM x 128 lanes x 2 x 1.965 GHz)"
        elif mode == "fp32x3" and args.op == "fwd":
            peak, peak_note = peaks["bf16_tflops"] / 6, f"a sixth of the {peaks['source']} bf16 burst peak (three tf32 products per multiply)"
        elif mode == "tf32":
            peak, peak_note = peaks["bf16_tflops"] / 2, f"half of the {peaks['source']} bf16 burst peak"
        else:
            peak, peak_note = peaks["bf16_tflops"], f"{peaks['source']} cuBLAS bf16 burst peak"
        line = {
            "metric": METRIC if args.op == "fwd" else f"chebykan_layer_{args.op}_samples_per_s", "value": value,
            "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": {"bf16": "bf16", "tf32": "tf32", "fp32": "f32", "fp32x3": "tf32x3"}[mode],
            "data": "synthetic",
            "config": dict(CFG if not args.shape else {"workload": f"layer {args.op}, shape {args.shape}"},
                           batch_per_gpu=B, input_dim=n_in, output_dim=n_out, degree=deg, op=args.op,
                           global_batch=world * B, parallelism=f"dp{world} (rows sharded, no collective)",
                           l2_policy="inputs larger than L2 (x 268 MB + y 268 MB per step vs 126 MB L2)",
                           math_mode=mode),
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                         "frac": achieved / peak,
                         "traffic": TRAFFIC_BYTES.get(mode) if (args.op == "fwd" and not args.shape and not args.batch) else None,
                         "peak_note": peak_note,
                         "flops_per_launch": flops},
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": x_host.numel() * 4,
                    "d2h_bytes_per_step": y_host.numel() * 4, "steps": e2e_steps},
            "gpu_launches": args.steps,
            "clocks": clocks,
        }
        if world == 1 and not args.no_cpu_baseline:
            v, cores, times = cpu_reference_throughput(32768, 12.0)
            line["cpu_baseline"] = {"value": v, "unit": UNIT, "cores": cores, "kind": "port",
                                    "sample": f"32768 of 65536 rows per pass, best of {len(times)} passes "
                                              f"({sum(times):.1f} s of CPU work)"}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def cpu_model_baseline(cfg, max_seconds: float = 10.0):
    """The configuration's model built from the oracle's layer, timed on the host cores on a bounded batch."""
    import torch.nn as nn
    from kan_b200 import workloads
    from oracle import chebykan_oracle as o

    class OracleLayer(nn.Module):
        def __init__(self, input_dim, output_dim, degree):
            super().__init__()
            self.input_dim = input_dim
            self.cheby_coeffs = nn.Parameter(o.init_coeffs(input_dim, output_dim, degree))

        def forward(self, x):
            return o.forward(x.view(-1, self.input_dim), self.cheby_coeffs)

    torch.set_num_threads(os.cpu_count() or 1)
    rows = {"cfg1": 100, "cfg2": 256, "cfg4": 2048, "cfg5": 32768}[cfg.name]
    model = workloads.build_model(cfg, OracleLayer)
    x, tgt = workloads.make_inputs(cfg, batch=rows)
    train = cfg.task == "train"
    if train:
        loss_fn = workloads.loss_fn(cfg)
        opt = (torch.optim.Adam if cfg.optimizer == "adam" else torch.optim.SGD)(model.parameters(), lr=cfg.lr)

        def step():
            opt.zero_grad()
            loss_fn(model(x), tgt).backward()
            opt.step()
    else:
        def step():
            with torch.no_grad():
                model(x)
    step()
    times = []
    while sum(times) < max_seconds and len(times) < 2000:
        t0 = time.perf_counter()
        step()
        times.append(time.perf_counter() - t0)
    best = min(times)
    return {"value": rows / best, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
            "ms_per_step": best * 1e3,
            "sample": f"{rows} of {cfg.batch} rows per step, best of {len(times)} steps ({sum(times):.1f} s of CPU work)"}


def run_model_config(args):
    """Other configurations (not the headline): one step = one forward pass (cfg4) or one
    forward + backward + optimizer step (cfg1, cfg2, cfg5) of the configuration's model."""
    import torch.distributed as dist
    import kan_b200
    from kan_b200 import dp, ops, workloads

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    cfg = workloads.CONFIGS[args.config]
    B = args.batch or cfg.batch
    mode = args.mode
    train = cfg.task == "train"
    model = workloads.build_model(cfg, kan_b200.ChebyKANLayer, math_mode=mode).to(dev)
    x, tgt = workloads.make_inputs(cfg, batch=B, seed=cfg.seed + rank)
    x = x.to(dev)
    tgt = tgt.to(dev) if tgt is not None else None
    n_cheby = len(cfg.layers)
    if train and args.graph:
        # the whole step (forward, loss, backward, optimizer) replayed as one CUDA graph
        if world > 1:
            raise SystemExit("--graph is a single-GPU mode")
        loss_fn = workloads.loss_fn(cfg)
        if cfg.optimizer == "adam":
            opt = kan_b200.optim.Adam(list(model.parameters()), lr=cfg.lr, capturable=True)
        else:
            opt = kan_b200.optim.SGD(list(model.parameters()), lr=cfg.lr)
        graphed = kan_b200.graph.GraphedTrainStep(model, loss_fn, opt, x, tgt)
        last_loss = [None]

        def step():
            last_loss[0] = graphed()
    elif train:
        loss_fn = workloads.loss_fn(cfg)
        buf = dp.FlatGradBuffer(model.parameters())
        Opt = kan_b200.optim.Adam if cfg.optimizer == "adam" else kan_b200.optim.SGD
        opt = Opt(list(model.parameters()), lr=cfg.lr)
        opt.grad_scale = 1.0 / world
        last_loss = [None]

        def step():
            buf.zero()
            loss = loss_fn(model(x), tgt)
            loss.backward()
            buf.all_reduce()
            opt.step()
            last_loss[0] = loss
    else:
        for p in model.parameters():
            p.requires_grad_(False)
        runner = kan_b200.fuse_layernorm(model) if (args.fuse_ln and mode not in ("fp32", "fp32x3")) else model

        def step():
            with torch.no_grad():
                runner(x)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    sampler = ClockSampler(local) if rank == 0 else None
    if sampler:
        sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    ev0.record()
    for _ in range(args.steps):
        step()
    ev1.record()
    barrier()
    clocks = sampler.stop() if sampler else None
    ops.check_status()
    t = torch.tensor([ev0.elapsed_time(ev1)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step = float(t.item()) / args.steps
    value = world * B / (ms_step * 1e-3)
    if rank == 0:
        peaks = measured_peaks()
        fwd_flops = workloads.flops_per_sample(cfg) * B
        # training: forward + dC for every layer + dx for every layer but the first
        later = sum(2 * i * (d + 1) * o for i, o, d in cfg.layers[1:]) * B
        flops = (2 * fwd_flops + later) if train else fwd_flops
        achieved = flops / (ms_step * 1e-3) / 1e12
        peak = peaks["bf16_tflops"] if (mode == "bf16" and not train) else (
            peaks["bf16_tflops"] / 2 if mode != "fp32" else 148 * 128 * 2 * 1.965e9 / 1e12)
        launches = n_cheby * (1 if not train else 6) + (len(list(model.parameters())) if train else 0)
        line = {
            "metric": "chebykan_%s_samples_per_s" % ("train_step" if train else "stack_fwd"), "value": value,
            "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": {"bf16": "bf16", "tf32": "tf32", "fp32": "f32", "fp32x3": "tf32x3"}[mode], "data": "synthetic",
            "config": {"workload": f"{cfg.name}: layers {list(cfg.layers)}, batch {B} per GPU, "
                                   f"{'fwd+bwd+' + cfg.optimizer if train else 'forward'}",
                       "global_batch": world * B, "math_mode": mode, "cuda_graph": bool(args.graph and train),
                       "layernorm_fused": bool(args.fuse_ln and not train and mode not in ("fp32", "fp32x3")),
                       "parallelism": f"dp{world}" + (" (flat-buffer all-reduce of the gradients)" if train and world > 1 else "")},
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                         "frac": achieved / peak, "traffic": None, "flops_per_step": flops},
            "gpu_launches": args.steps * launches, "clocks": clocks,
        }
        if train:
            line["final_loss"] = float(last_loss[0].detach())
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_model_baseline(cfg)
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


# DRAM bytes (read + write) of one forward launch taken from an ncu capture; None until one exists.
# bf16/tf32/fp32: captured at 32768 rows (profiles/), x and y traffic doubled for the full 65536-row launch;
# fp32x3: captured at 16384 rows, x and y traffic times four (x is re-read once per 256-column tile).
TRAFFIC_BYTES = {"bf16": 572.1e6, "tf32": 768.9e6, "fp32": 592.4e6, "fp32x3": 1505.5e6}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--mode", default="bf16", choices=["bf16", "tf32", "fp32", "fp32x3"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end leg (profiling runs)")
    ap.add_argument("--batch", type=int, default=0, help="rows per GPU (default: the configuration's batch)")
    ap.add_argument("--fuse-ln", action="store_true",
                    help="forward stacks: fold the LayerNorms between layers into the ChebyKAN kernels")
    ap.add_argument("--graph", action="store_true",
                    help="training configurations: replay the whole step as one CUDA graph (single GPU)")
    ap.add_argument("--op", default="fwd", choices=["fwd", "dcoeff", "dx"],
                    help="cfg3 path only: time the forward (headline) or one backward kernel on the same shape")
    ap.add_argument("--shape", default="", help="cfg3 path only: B,in,out,deg override (profiling other layer shapes)")
    ap.add_argument("--config", default="cfg3", choices=["cfg1", "cfg2", "cfg3", "cfg4", "cfg5"],
                    help="cfg3 (default) is the headline forward; the others time the configuration's model step")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.config != "cfg3":
        run_model_config(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
