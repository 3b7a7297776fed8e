#!/usr/bin/env python
"""Benchmark of the ChebyKAN layer hot path on B200.

    python bench.py --gpus N --steps K --warmup W          # this library (one rank per GPU under torch.distributed.run)
    python bench.py --impl reference --gpus N ...         # the reference's CPU path on the host cores (rank 0 only)

Headline (the JSON line's `value`): forward of configuration 3, one ChebyKANLayer 1024 -> 1024 of degree 8 on a
GLOBAL batch of 65536 rows, bf16-stored coefficients.  With N > 1 the rows are sharded over the ranks
(`dp.shard_rows`, no collective: rows are independent), so `scaling` is "strong" and `value` = 65536 rows /
max-over-ranks time per step.  One "step" is one forward pass over the (sharded) batch.

The same line carries, under `sub`, the other configurations and modes measured in the same process:
the weak-scaling forward (a full batch per GPU), configuration 4's four-layer stack (32768 rows, sharded),
configuration 5's training step (1048576 rows, sharded, fused MSE loss, NCCL all-reduce of the coefficient
gradients, SGD) and, on one GPU, the tf32 / fp32x3 / fp32 forwards, the backward kernels, a sustained run and the
launch-bound configurations 1 and 2.  `--no-sub` skips them; the profiling flags (`--batch`, `--shape`, `--op`,
`--config`) select a single measurement instead.

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
CFG3 = dict(global_batch=65536, input_dim=1024, output_dim=1024, degree=8)
DTYPE_NAME = {"bf16": "bf16", "tf32": "tf32", "fp32": "f32", "fp32x3": "tf32x3"}
L2_BYTES = 126 << 20
FFMA_PEAK_TFLOPS = 148 * 128 * 2 * 1.965e9 / 1e12      # nominal: 148 SMs x 128 FFMA lanes x 2 FLOP x 1.965 GHz


def headline_config(world: int) -> dict:
    """The workload description both arms print (the reference arm times the same 65536-row step on the host)."""
    return {"workload": "cfg3: ChebyKANLayer fwd, global batch 65536, in=1024, out=1024, degree=8, x~N(0,1) fp32, "
                        "coefficients ~ N(0, 1/(1024*9))",
            "global_batch": CFG3["global_batch"], "input_dim": CFG3["input_dim"], "output_dim": CFG3["output_dim"],
            "degree": CFG3["degree"], "n_gpus": world,
            "parallelism": f"dp{world}: rows sharded over the GPUs, coefficients replicated, no collective in inference",
            "l2_policy": "x + y per GPU = 537 MB / N: larger than twice the 126 MB L2 up to 2 GPUs, timed back to back; "
                         "from 4 GPUs on every timed step has its own event pair and a 256 MB buffer is overwritten "
                         "between steps (L2 flush)"}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm_gbs=p["hbm_gbs"], bf16_tflops=p["bf16_tflops"],
                    bf16_tflops_sustained=p.get("bf16_tflops_sustained"), source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


def measured_traffic(key: str, rows: int):
    """DRAM bytes of one launch from the committed ncu capture `key` (profiles/traffic.json, written by
    `python -m kan_b200.ncu_summary`), scaled from the captured rows to `rows`: the per-row part grows with the
    batch, the coefficients do not.  None when no capture of that kernel is on record."""
    path = os.path.join(ROOT, "profiles", "traffic.json")
    if not os.path.exists(path):
        return None
    with open(path) as f:
        rec = json.load(f).get(key)
    if not rec:
        return None
    fixed = rec.get("fixed_bytes", 0.0)
    per_row = (rec["dram_bytes_per_launch"] - fixed) / rec["rows_captured"]
    return {"bytes": per_row * rows + fixed, "capture": key, "rows_captured": rec["rows_captured"]}


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
        return self

    def stop(self):
        if self._thr is not None:
            self._stop.set()
            self._thr.join()
        med = statistics.median(self.samples) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


# ----------------------------------------------------------------------------------------------
# reference arm: the reference's own CPU implementation of the path on the host cores
# ----------------------------------------------------------------------------------------------
def reference_forward_fn():
    """(forward(x) -> y, kind, description): the unmodified reference layer when its tree is found (the directory in
    $KAN_REF, baseline/_ref/ or the build container's read-only mount), else the op-for-op restatement."""
    from oracle import chebykan_oracle as o
    from oracle import ref_loader
    torch.manual_seed(1003)
    if ref_loader.available():
        try:
            Layer = ref_loader.reference_layer_cls()
            layer = Layer(CFG3["input_dim"], CFG3["output_dim"], CFG3["degree"])

            def fwd(x):
                with torch.no_grad():
                    return layer(x)
            return fwd, "reference", "kan.layers.chebykan.ChebyKANLayer (unmodified, closed-form basis + einsum, torch CPU fp32)"
        except Exception:       # a tree that does not import falls back to the restatement
            pass
    coeffs = o.init_coeffs(CFG3["input_dim"], CFG3["output_dim"], CFG3["degree"])

    def fwd(x):
        with torch.no_grad():
            return o.forward(x, coeffs)
    return fwd, "port", "op-for-op restatement of the reference layer (closed-form basis + einsum, torch CPU fp32)"


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    world = int(os.environ.get("WORLD_SIZE", str(args.gpus)))
    torch.set_num_threads(os.cpu_count() or 1)
    rows = args.batch or CFG3["global_batch"]          # the same rows per step as the GPU arm
    fwd, kind, what = reference_forward_fn()
    g = torch.Generator().manual_seed(1003)
    x = torch.randn(rows, CFG3["input_dim"], generator=g)
    fwd(x[:256])                                        # warm the thread pool
    for _ in range(args.warmup):
        fwd(x)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        fwd(x)
    dt = time.perf_counter() - t0
    value = rows * args.steps / dt
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": headline_config(world),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": torch.get_num_threads(), "kind": kind,
                         "sample": f"{rows} rows per step, {args.steps} steps: {what}"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


def cpu_baseline_cfg3(max_seconds: float = 12.0):
    """cpu_baseline of the GPU arm: the same 65536-row step on the host cores, best of a few passes."""
    torch.set_num_threads(os.cpu_count() or 1)
    fwd, kind, what = reference_forward_fn()
    rows = CFG3["global_batch"]
    x = torch.randn(rows, CFG3["input_dim"], generator=torch.Generator().manual_seed(1003))
    fwd(x[:256])
    times = []
    while sum(times) < max_seconds and len(times) < 20:
        t0 = time.perf_counter()
        fwd(x)
        times.append(time.perf_counter() - t0)
    return {"value": rows / min(times), "unit": UNIT, "cores": torch.get_num_threads(), "kind": kind,
            "sample": f"{rows} rows per pass (the whole step), best of {len(times)} passes "
                      f"({sum(times):.1f} s of CPU work): {what}"}


def cpu_model_baseline(cfg, max_seconds: float = 8.0):
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


# ----------------------------------------------------------------------------------------------
# GPU arm
# ----------------------------------------------------------------------------------------------
class Ctx:
    """Rank, device and the barrier / max-over-ranks timing every measurement uses."""

    def __init__(self):
        import torch.distributed as dist
        self.dist = dist
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(self.local)
        self.dev = torch.device("cuda", self.local)
        self._flush = None
        if self.world > 1:
            dist.init_process_group("nccl", device_id=self.dev)

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(self, v: float) -> float:
        t = torch.tensor([v], dtype=torch.float64, device=self.dev)
        if self.world > 1:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def time_steps(self, step, steps: int, warmup: int, sample_clocks: bool = False, flush_l2: bool = False):
        """ms per step: `warmup` untimed steps, then exactly `steps` steps between CUDA events on the launching
        stream, a barrier + synchronize on both sides, max over ranks.  With `flush_l2` (working sets that would
        fit the 126 MB L2) every step gets its own event pair and a 256 MB buffer is overwritten between the pairs,
        so no step finds its inputs in L2; the step times are added up."""
        from kan_b200 import ops
        for _ in range(max(warmup, 3)):
            step()
        self.barrier()
        sampler = ClockSampler(self.local).start() if (sample_clocks and self.rank == 0) else None
        if flush_l2:
            if self._flush is None:
                self._flush = torch.empty(256 << 20, dtype=torch.uint8, device=self.dev)
            evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
            self.barrier()
            self._flush.zero_()
            step()                      # untimed: lets the host run ahead of the GPU before the first timed pair
            for a, b in evs:
                self._flush.zero_()
                a.record()
                step()
                b.record()
            self.barrier()
            total = sum(a.elapsed_time(b) for a, b in evs)
        else:
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            self.barrier()
            ev0.record()
            for _ in range(steps):
                step()
            ev1.record()
            self.barrier()
            total = ev0.elapsed_time(ev1)
        clocks = sampler.stop() if sampler else None
        ops.check_status()
        ms = self.max_over_ranks(total) / steps
        return ms, clocks

    def close(self):
        if self.world > 1:
            self.dist.destroy_process_group()


def free_gpu():
    import gc
    gc.collect()
    torch.cuda.empty_cache()


def tensor_peak(mode: str, op: str, peaks: dict, tf32_peak, n_out: int = 0):
    """(peak TFLOP/s, note) a kernel of this mode is quoted against.  dC contracts tf32 (or, on narrow layers, fp16)
    operands in both tensor-core modes; dx does too, except in bf16 mode on layers of 512 outputs or more, where it
    contracts fp16 operands and is quoted against the 16-bit peak."""
    if mode == "fp32":
        return FFMA_PEAK_TFLOPS, "nominal FFMA peak (148 SM x 128 lanes x 2 x 1.965 GHz)"
    tf32 = tf32_peak["tflops"] if tf32_peak else peaks["bf16_tflops"] / 2
    tf32_note = ("tf32 peak measured in this run (torch.matmul 8192^3, allow_tf32, best of 10)" if tf32_peak
                 else f"half of the {peaks['source']} bf16 burst peak (no tf32 measurement in this run)")
    if mode == "fp32x3":
        return tf32 / 3, "a third of the " + tf32_note + ": three tf32 products per multiply"
    if op == "dx" and mode == "bf16" and n_out >= 512:
        return peaks["bf16_tflops"], f"{peaks['source']} cuBLAS bf16 burst peak (fp16 operands)"
    if mode == "tf32" or op in ("dcoeff", "dx"):
        return tf32, tf32_note
    return peaks["bf16_tflops"], f"{peaks['source']} cuBLAS bf16 burst peak"


def measure_tf32_peak(dev):
    """cuBLAS tf32 GEMM rate the way MEASURED_PEAKS.json measures bf16: torch.matmul 8192^3, best of 10, CUDA events.
    Outside every timed region; restores the allow_tf32 switch."""
    n = 8192
    a = torch.randn(n, n, device=dev)
    b = torch.randn(n, n, device=dev)
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = True
    try:
        for _ in range(3):
            torch.matmul(a, b)
        best = float("inf")
        for _ in range(10):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            torch.matmul(a, b)
            e1.record()
            torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1))
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev
    del a, b
    free_gpu()
    return {"tflops": 2.0 * n ** 3 / (best * 1e-3) / 1e12, "how": "torch.matmul fp32 8192^3 with allow_tf32, best of 10"}


def measure_host_link(ctx: Ctx, bytes_in: int, bytes_out: int, reps: int = 5):
    """Ceiling of the end-to-end figure: plain pinned cudaMemcpyAsync of the same bytes, host-to-device and
    device-to-host at the same time on two streams, all ranks at once; ms per step, max over ranks."""
    hin = torch.empty(bytes_in, dtype=torch.uint8).pin_memory()
    hout = torch.empty(bytes_out, dtype=torch.uint8).pin_memory()
    din = torch.empty(bytes_in, dtype=torch.uint8, device=ctx.dev)
    dout = torch.empty(bytes_out, dtype=torch.uint8, device=ctx.dev)
    s1, s2 = torch.cuda.Stream(ctx.dev), torch.cuda.Stream(ctx.dev)

    def once():
        cur = torch.cuda.current_stream(ctx.dev)
        s1.wait_stream(cur)
        s2.wait_stream(cur)
        with torch.cuda.stream(s1):
            din.copy_(hin, non_blocking=True)
        with torch.cuda.stream(s2):
            hout.copy_(dout, non_blocking=True)
        cur.wait_stream(s1)
        cur.wait_stream(s2)
    once()
    ctx.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        once()
    e1.record()
    ctx.barrier()
    ms = ctx.max_over_ranks(e0.elapsed_time(e1)) / reps
    del hin, hout, din, dout
    free_gpu()
    return ms


def bench_layer(ctx: Ctx, mode: str, op: str, B: int, n_in: int, n_out: int, deg: int, steps: int, warmup: int,
                sample_clocks: bool = False, seed_offset: int = 0, family: str = ""):
    """One kernel of one layer on `B` resident rows per rank; returns (ms per step, clocks, state for e2e).
    `family` ('jacobi', 'hermite', 'hermite_prob'): the same kernel with that family's recurrence table."""
    import kan_b200
    from kan_b200 import ops
    torch.manual_seed(1003)
    layer = kan_b200.ChebyKANLayer(n_in, n_out, deg, math_mode=mode).to(ctx.dev)
    for p in layer.parameters():
        p.requires_grad_(False)
    g = torch.Generator().manual_seed(1003 + seed_offset)
    x_host = torch.randn(B, n_in, generator=g)
    x = x_host.to(ctx.dev)
    packed = ops.pack_coeffs(layer.cheby_coeffs.detach(), mode)
    fam = ops.make_family(family, alpha=0.5, beta=-0.3) if family else None     # (alpha, beta) matter to Jacobi only
    if op == "fwd":
        y = torch.empty(B, n_out, dtype=torch.float32, device=ctx.dev)

        def step():
            if fam is not None:
                ops.family_forward(fam, x, packed, n_in, n_out, deg, mode, out=y)
            else:
                ops.forward(x, packed, n_in, n_out, deg, mode, out=y)
    else:
        dy = torch.randn(B, n_out, device=ctx.dev)
        cdev = layer.cheby_coeffs.detach()
        if op == "dcoeff":
            dc = torch.empty(n_in, n_out, deg + 1, device=ctx.dev)

            def step():
                if fam is not None:
                    ops.family_bwd_dcoeff(fam, x, dy, n_in, n_out, deg, mode, out=dc)
                else:
                    ops.bwd_dcoeff(x, dy, n_in, n_out, deg, mode, out=dc)
        else:
            dx = torch.empty(B, n_in, device=ctx.dev)

            def step():
                if fam is not None:
                    ops.family_bwd_dx(fam, x, dy, cdev, mode, out=dx)
                else:
                    ops.bwd_dx(x, dy, cdev, mode, out=dx)
    flush = B * 4 * (n_in + n_out) < 2 * L2_BYTES
    ms, clocks = ctx.time_steps(step, steps, warmup, sample_clocks, flush_l2=flush)
    return ms, clocks, dict(layer=layer, x_host=x_host, step=step, flushed=flush)


def sub_layer_fwd_bwd(ctx: Ctx, mode: str, B: int, n_in: int, n_out: int, deg: int, steps: int, warmup: int):
    """Forward and backward of ONE layer through the drop-in module and autograd (y = layer(x); y.backward(dY) with
    x requiring a gradient, so that both dC and dx are computed), B resident rows per rank: the 'fwd+bwd ms/step' of a
    wide layer.  FLOPs counted as three products of 2*B*in*(deg+1)*out."""
    import kan_b200
    torch.manual_seed(1003)
    layer = kan_b200.ChebyKANLayer(n_in, n_out, deg, math_mode=mode).to(ctx.dev)
    g = torch.Generator().manual_seed(1004 + ctx.rank)
    x = torch.randn(B, n_in, generator=g).to(ctx.dev).requires_grad_(True)
    dy = torch.randn(B, n_out, generator=g).to(ctx.dev)

    def step():
        x.grad = None
        layer.cheby_coeffs.grad = None
        layer(x).backward(dy)
    ms, _ = ctx.time_steps(step, steps, warmup)
    flops = 3 * 2.0 * B * n_in * (deg + 1) * n_out
    rec = {"workload": f"one ChebyKANLayer {n_in}->{n_out} degree {deg}, {B} rows per GPU: forward + backward (dC and dx) "
                       "through torch autograd",
           "value": B * ctx.world / (ms * 1e-3), "unit": UNIT, "ms_per_step": ms, "rows_per_gpu": B, "math_mode": mode,
           "operands": {"fwd": mode, "dcoeff": "tf32", "dx": "f16" if (mode == "bf16" and n_out >= 512) else "tf32"},
           "achieved_tflops": flops / (ms * 1e-3) / 1e12}
    del layer, x, dy
    free_gpu()
    return rec


def layer_record(ctx, mode, op, B_rank, B_total, shape, ms, peaks, tf32_peak, extra=None):
    n_in, n_out, deg = shape
    flops_rank = 2.0 * B_rank * n_in * (deg + 1) * n_out
    achieved = flops_rank / (ms * 1e-3) / 1e12
    peak, note = tensor_peak(mode, op, peaks, tf32_peak, n_out)
    rec = {"value": B_total / (ms * 1e-3), "unit": UNIT, "ms_per_step": ms, "rows_per_gpu": B_rank,
           "dtype": "f16" if (op == "dx" and mode == "bf16" and n_out >= 512) else DTYPE_NAME[mode],
           "roofline": {"bound": "tensor" if mode != "fp32" else "ffma", "achieved": achieved, "peak": peak,
                        "unit": "TFLOP/s", "frac": achieved / peak, "peak_note": note}}
    if extra:
        rec.update(extra)
    return rec


def sub_family(ctx: Ctx, kind: str, B: int, n_in: int, n_out: int, deg: int, peaks, **family_kw):
    """Forward (fp32 FFMA kernel and bf16 tensor-core kernel), dC and dx (fp32 FFMA kernels and tf32 tensor-core kernels)
    of a Jacobi / Hermite layer, all with a table-driven recurrence, on B resident rows of this rank; ms per launch and
    the rate of each against its pipe."""
    from kan_b200 import ops
    fam = ops.make_family(kind, **family_kw)
    g = torch.Generator().manual_seed(77 + ctx.rank)
    x = torch.randn(B, n_in, generator=g).to(ctx.dev)
    dy = torch.randn(B, n_out, generator=g).to(ctx.dev)
    coeffs = (torch.randn(n_in, n_out, deg + 1, generator=g) / (n_in * (deg + 1))).to(ctx.dev)
    packed = ops.pack_coeffs(coeffs, "fp32")
    y, dc, dx = torch.empty(B, n_out, device=ctx.dev), torch.empty_like(coeffs), torch.empty_like(x)
    packed_bf16 = ops.pack_coeffs(coeffs, "bf16")
    steps = {"fwd": lambda: ops.family_forward(fam, x, packed, n_in, n_out, deg, "fp32", out=y),
             "fwd_bf16": lambda: ops.family_forward(fam, x, packed_bf16, n_in, n_out, deg, "bf16", out=y),
             "dcoeff": lambda: ops.family_bwd_dcoeff(fam, x, dy, n_in, n_out, deg, "fp32", out=dc),
             "dx": lambda: ops.family_bwd_dx(fam, x, dy, coeffs, "fp32", out=dx),
             "dcoeff_tf32": lambda: ops.family_bwd_dcoeff(fam, x, dy, n_in, n_out, deg, "tf32", out=dc),
             "dx_tf32": lambda: ops.family_bwd_dx(fam, x, dy, coeffs, "tf32", out=dx)}
    flops = 2.0 * B * n_in * (deg + 1) * n_out
    rec = {"family": dict(family_kw, kind=kind), "rows_per_gpu": B, "shape": [n_in, n_out, deg], "dtype": "fp32"}
    for op, fn in steps.items():
        ms, _ = ctx.time_steps(fn, 3, 3, False, flush_l2=B * 4 * (n_in + n_out) < 2 * L2_BYTES)
        tc_mode = {"fwd_bf16": "bf16", "dcoeff_tf32": "tf32", "dx_tf32": "tf32"}.get(op)
        peak, note = tensor_peak(tc_mode or "fp32", "fwd", peaks, None)
        rec[op] = {"ms_per_step": ms, "value": B * ctx.world / (ms * 1e-3), "unit": UNIT,
                   "roofline": {"bound": "tensor" if tc_mode else "ffma", "achieved": flops / (ms * 1e-3) / 1e12, "peak": peak, "unit": "TFLOP/s",
                                "frac": flops / (ms * 1e-3) / 1e12 / peak, "peak_note": note}}
    ops.check_status()
    del x, dy, coeffs, packed, packed_bf16, y, dc, dx
    free_gpu()
    return rec


def sub_sustained(ctx: Ctx, state, B: int, peaks: dict, seconds: float = 2.0):
    """Back-to-back launches for `seconds`: the clock settles under the power limit.  Quoted against the sustained
    cuBLAS figure, with time x median SM clock beside it."""
    step = state["step"]
    for _ in range(3):
        step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    step()
    e0.record(); step(); e1.record()
    torch.cuda.synchronize()
    n = max(50, int(seconds * 1e3 / max(e0.elapsed_time(e1), 1e-3)))
    sampler = ClockSampler(ctx.local).start()
    e0.record()
    for _ in range(n):
        step()
    e1.record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    ms = e0.elapsed_time(e1) / n
    flops = 2.0 * B * CFG3["input_dim"] * (CFG3["degree"] + 1) * CFG3["output_dim"]
    achieved = flops / (ms * 1e-3) / 1e12
    peak = peaks.get("bf16_tflops_sustained") or peaks["bf16_tflops"]
    return {"value": B / (ms * 1e-3), "unit": UNIT, "ms_per_step": ms, "launches": n, "seconds": ms * n / 1e3,
            "clocks": clocks, "ms_times_sm_mhz": (ms * clocks["sm_mhz"]) if clocks and clocks["sm_mhz"] else None,
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                         "peak_note": f"{peaks['source']} cuBLAS bf16 rate sustained over seconds under the power cap"}}


def sub_stack_cfg4(ctx: Ctx, mode: str, fuse_ln: bool, steps: int, warmup: int, peaks, tf32_peak, batch: int = 0):
    import kan_b200
    from kan_b200 import dp, workloads
    cfg = workloads.CONFIGS["cfg4"]
    Bg = batch or cfg.batch
    b, e = dp.shard_rows(Bg, ctx.rank, ctx.world)
    model = workloads.build_model(cfg, kan_b200.ChebyKANLayer, math_mode=mode).to(ctx.dev)
    for p in model.parameters():
        p.requires_grad_(False)
    x, _ = workloads.make_inputs(cfg, batch=Bg)
    x = x[b:e].contiguous().to(ctx.dev)
    runner = kan_b200.fuse_layernorm(model) if fuse_ln else model

    def step():
        with torch.no_grad():
            runner(x)
    ms, _ = ctx.time_steps(step, steps, warmup)
    flops_rank = workloads.flops_per_sample(cfg) * (e - b)
    achieved = flops_rank / (ms * 1e-3) / 1e12
    peak, note = tensor_peak(mode, "fwd", peaks, tf32_peak)
    rec = {"workload": f"cfg4: 4 x ChebyKANLayer 2048->2048 degree 4 with LayerNorm between, global batch {Bg}, forward",
           "value": Bg / (ms * 1e-3), "unit": UNIT, "ms_per_step": ms, "rows_per_gpu": e - b, "dtype": DTYPE_NAME[mode],
           "layernorm_fused": fuse_ln, "scaling": "strong",
           "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                        "peak_note": note}}
    del model, runner, x
    free_gpu()
    return rec


def sub_train_cfg5(ctx: Ctx, mode: str, steps: int, warmup: int, peaks, tf32_peak, batch: int = 0, torch_loss: bool = False,
                   graph: bool = False):
    """Configuration 5: 64 -> 64 -> 64, degree 32, global batch 1048576 sharded over the ranks; forward, MSE loss
    (mean over the GLOBAL batch), backward, NCCL all-reduce of the flat gradient buffer, SGD.  With `graph` the
    whole step, collective included, is recorded once and replayed as one CUDA graph per rank (the host needs
    about 0.5 ms to issue the step's launches, more than the kernels take once the batch is split eight ways)."""
    import kan_b200
    from kan_b200 import dp, ops, workloads
    cfg = workloads.CONFIGS["cfg5"]
    Bg = batch or cfg.batch
    b, e = dp.shard_rows(Bg, ctx.rank, ctx.world)
    model = workloads.build_model(cfg, kan_b200.ChebyKANLayer, math_mode=mode).to(ctx.dev)
    g = torch.Generator().manual_seed(cfg.seed + ctx.rank)
    x = torch.rand(e - b, cfg.layers[0][0], generator=g) * 6.0 - 3.0
    tgt = torch.sin(x).sum(1, keepdim=True).expand(-1, cfg.layers[-1][1]).contiguous()
    x, tgt = x.to(ctx.dev), tgt.to(ctx.dev)
    buf = dp.FlatGradBuffer(model.parameters())
    opt = kan_b200.optim.SGD(list(model.parameters()), lr=cfg.lr)
    n_mean = Bg * cfg.layers[-1][1]
    if torch_loss:
        opt.grad_scale = 1.0 / ctx.world
        mse = torch.nn.MSELoss()
    last = {}
    ar0 = [torch.cuda.Event(enable_timing=True) for _ in range(steps + max(warmup, 3))]
    ar1 = [torch.cuda.Event(enable_timing=True) for _ in range(steps + max(warmup, 3))]
    k = [0]

    def step():
        buf.zero()
        y = model(x)
        loss = mse(y, tgt) if torch_loss else kan_b200.mse_loss(y, tgt, n_mean=n_mean)
        loss.backward()
        i = k[0] % len(ar0)
        ar0[i].record()
        buf.all_reduce()
        ar1[i].record()
        opt.step()
        last["loss"] = loss
        k[0] += 1
    if graph:
        graphed = kan_b200.graph.GraphedTrainStep(model, lambda y_, t_: kan_b200.mse_loss(y_, t_, n_mean=n_mean), opt,
                                                  x, tgt)
        buf = graphed.grads

        def step():                                            # noqa: F811 - the replayed step replaces the eager one
            last["loss"] = graphed()
    ms, _ = ctx.time_steps(step, steps, warmup)
    torch.cuda.synchronize()
    w = max(warmup, 3)
    ar_ms = None if graph else ctx.max_over_ranks(sum(ar0[w + i].elapsed_time(ar1[w + i]) for i in range(steps)) / steps)
    loss = last["loss"].detach().clone()
    if ctx.world > 1 and not torch_loss:
        ctx.dist.all_reduce(loss)          # per-rank partial sums of the global mean
    rows = e - b
    fwd = workloads.flops_per_sample(cfg) * rows
    later = sum(2 * i * (d + 1) * o_ for i, o_, d in cfg.layers[1:]) * rows
    flops_rank = 2 * fwd + later          # forward + dC for every layer + dx for every layer but the first
    achieved = flops_rank / (ms * 1e-3) / 1e12
    peak, note = tensor_peak("tf32", "fwd", peaks, tf32_peak)
    # algorithmic HBM bytes per row: x and y of each layer forward, x and dY of each dC, dY, x and dx of each dx,
    # output + target + dY of the loss
    hbm_bytes = rows * 4.0 * (sum(i + o_ for i, o_, _ in cfg.layers) * 2 + sum(2 * o_ + i for i, o_, _ in cfg.layers[1:])
                               + 3 * cfg.layers[-1][1])
    rec = {"workload": f"cfg5: ChebyKAN 64->64->64 degree 32, global batch {Bg}, fwd + MSE + bwd + all-reduce(dC) + SGD",
           "value": Bg / (ms * 1e-3), "unit": UNIT, "ms_per_step": ms, "rows_per_gpu": rows, "math_mode": mode,
           "loss": "torch.nn.MSELoss" if torch_loss else "kan_b200.mse_loss (loss and gradient in one pass)",
           "scaling": "strong", "allreduce_ms": ar_ms if ctx.world > 1 else 0.0, "cuda_graph": bool(graph),
           "allreduce_bytes": buf.flat.numel() * 4, "final_loss": float(loss),
           "roofline": {"bound": "basis generation / stage hand-over (neither tensor- nor HBM-bound)",
                        "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                        "peak_note": "GEMM-equivalent FLOPs (fwd + dC per layer, dx for the second) against the " + note,
                        "hbm_gbs": hbm_bytes / (ms * 1e-3) / 1e9, "hbm_frac": hbm_bytes / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"]}}
    if graph:
        graphed.close()                 # a graph with a captured collective must be gone before the process group is
        del graphed, step
    del model, x, tgt, buf, opt
    free_gpu()
    return rec


def sub_small_train(ctx: Ctx, name: str, graph: bool, steps: int, warmup: int, fused: bool = False):
    """Launch-bound configurations 1 and 2 (single GPU): ms per training step, eager, replayed as one CUDA graph, or
    (configuration 1: one layer, MSE) as the single-launch fused step."""
    import kan_b200
    from kan_b200 import dp, workloads
    cfg = workloads.CONFIGS[name]
    model = workloads.build_model(cfg, kan_b200.ChebyKANLayer, math_mode="fp32").to(ctx.dev)
    x, tgt = workloads.make_inputs(cfg)
    x, tgt = x.to(ctx.dev), tgt.to(ctx.dev)
    loss_fn = workloads.loss_fn(cfg)
    if fused:
        fused_step = kan_b200.small.FusedTrainStep(model[0], cfg.optimizer, lr=cfg.lr)

        def step():
            fused_step(x, tgt)
    elif graph:
        opt = (kan_b200.optim.Adam(list(model.parameters()), lr=cfg.lr, capturable=True) if cfg.optimizer == "adam"
               else kan_b200.optim.SGD(list(model.parameters()), lr=cfg.lr))
        graphed = kan_b200.graph.GraphedTrainStep(model, loss_fn, opt, x, tgt)
        step = graphed
    else:
        buf = dp.FlatGradBuffer(model.parameters())
        Opt = kan_b200.optim.Adam if cfg.optimizer == "adam" else kan_b200.optim.SGD
        opt = Opt(list(model.parameters()), lr=cfg.lr)

        def step():
            buf.zero()
            loss_fn(model(x), tgt).backward()
            opt.step()
    ms, _ = ctx.time_steps(step, steps, warmup)
    rec = {"workload": f"{name}: layers {list(cfg.layers)}, batch {cfg.batch}, fwd+bwd+{cfg.optimizer}, fp32",
           "value": cfg.batch / (ms * 1e-3), "unit": UNIT, "ms_per_step": ms, "cuda_graph": graph,
           "single_launch_step": fused, "roofline": {"bound": "launch latency"}}
    free_gpu()
    return rec


def run_ours(args):
    from kan_b200 import dp, ops
    ctx = Ctx()
    peaks = measured_peaks()
    n_in, n_out, deg = CFG3["input_dim"], CFG3["output_dim"], CFG3["degree"]
    Bg = args.batch or CFG3["global_batch"]
    if args.shape:
        Bg, n_in, n_out, deg = [int(v) for v in args.shape.split(",")]
    single = bool(args.shape or args.batch or args.op != "fwd" or args.family)      # a profiling run: one measurement only
    if args.family and args.mode == "fp32x3":
        raise SystemExit("--family runs in fp32, tf32 or bf16")
    mode = args.mode
    b, e = dp.shard_rows(Bg, ctx.rank, ctx.world)
    B = e - b
    tf32_peak = None
    if not single and not args.no_sub:
        tf32_peak = measure_tf32_peak(ctx.dev)        # every rank runs it (keeps the ranks in step); rank 0's is reported

    # ---- headline: strong-scaled forward, inputs resident
    ms_step, clocks, state = bench_layer(ctx, mode, args.op, B, n_in, n_out, deg, args.steps, args.warmup,
                                         sample_clocks=True, seed_offset=ctx.rank, family=args.family)
    value = Bg / (ms_step * 1e-3)
    flushed = state["flushed"]

    # ---- end to end through the layer's public host-buffer call: H2D of x, forward, D2H of y, pipelined
    e2e = None
    if args.op == "fwd" and not args.no_e2e and not args.family:
        layer, x_host = state["layer"], state["x_host"].pin_memory()
        y_host = torch.empty(B, n_out, dtype=torch.float32).pin_memory()
        e2e_steps = max(3, min(args.steps, 10))
        layer.forward_host(x_host, out=y_host)
        ctx.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(e2e_steps):
            layer.forward_host(x_host, out=y_host)
        e1.record()
        ctx.barrier()
        e2e_ms = ctx.max_over_ranks(e0.elapsed_time(e1)) / e2e_steps
        ops.check_status()
        link_ms = measure_host_link(ctx, x_host.numel() * 4, y_host.numel() * 4)
        e2e = {"value": Bg / (e2e_ms * 1e-3), "unit": UNIT, "h2d_bytes_per_step": x_host.numel() * 4 * ctx.world,
               "d2h_bytes_per_step": y_host.numel() * 4 * ctx.world, "steps": e2e_steps, "ms_per_step": e2e_ms,
               "link_ms_per_step": link_ms, "link_frac": link_ms / e2e_ms,
               "link_note": "link_ms = the same bytes as plain pinned cudaMemcpyAsync in both directions at once on all "
                            "ranks (the host link's ceiling for this step); link_frac = link_ms / e2e ms"}
        del y_host

    sub = {}
    if not single and not args.no_sub:
        ks, kw = max(3, min(args.steps, 10)), 3
        if ctx.world == 1:
            sub["cfg3_fwd_sustained_bf16"] = sub_sustained(ctx, state, B, peaks)
        del state
        free_gpu()
        if ctx.world > 1:
            ms, _, st = bench_layer(ctx, mode, "fwd", CFG3["global_batch"], n_in, n_out, deg, ks, kw, seed_offset=ctx.rank)
            del st
            free_gpu()
            sub["cfg3_fwd_weak_" + mode] = layer_record(
                ctx, mode, "fwd", CFG3["global_batch"], ctx.world * CFG3["global_batch"], (n_in, n_out, deg), ms, peaks,
                tf32_peak, {"scaling": "weak", "workload": "a full 65536-row batch on every GPU"})
        else:
            for m, op in (("tf32", "fwd"), ("fp32x3", "fwd"), ("fp32", "fwd"), ("tf32", "dcoeff"), ("tf32", "dx"),
                          ("bf16", "dx"), ("fp32x3", "dcoeff"), ("fp32x3", "dx")):
                ms, _, st = bench_layer(ctx, m, op, Bg, n_in, n_out, deg, ks if m != "fp32" else 3, kw)
                del st
                free_gpu()
                sub[f"cfg3_{op}_{m}"] = layer_record(ctx, m, op, Bg, Bg, (n_in, n_out, deg), ms, peaks, tf32_peak)
        if ctx.world == 1:
            sub["cfg3_fwd_bwd_bf16"] = sub_layer_fwd_bwd(ctx, "bf16", Bg, n_in, n_out, deg, ks, kw)
            sub["cfg3_fwd_bwd_tf32"] = sub_layer_fwd_bwd(ctx, "tf32", Bg, n_in, n_out, deg, ks, kw)
        sub["cfg4_stack_fwd_bf16"] = sub_stack_cfg4(ctx, "bf16", False, ks, kw, peaks, tf32_peak)
        sub["cfg4_stack_fwd_bf16_fused_ln"] = sub_stack_cfg4(ctx, "bf16", True, ks, kw, peaks, tf32_peak)
        sub["cfg5_train_tf32"] = sub_train_cfg5(ctx, "tf32", ks, kw, peaks, tf32_peak)
        sub["cfg5_train_bf16_fwd_tf32_bwd"] = sub_train_cfg5(ctx, "bf16", ks, kw, peaks, tf32_peak)
        sub["cfg5_train_tf32_graph"] = sub_train_cfg5(ctx, "tf32", ks, kw, peaks, tf32_peak, graph=True)
        if ctx.world == 1:
            sub["cfg5_train_tf32_torch_loss"] = sub_train_cfg5(ctx, "tf32", ks, kw, peaks, tf32_peak, torch_loss=True)
            sub["cfg5_train_fp32x3"] = sub_train_cfg5(ctx, "fp32x3", 3, kw, peaks, tf32_peak)
            sub["cfg3_shape_jacobi_fp32"] = sub_family(ctx, "jacobi", 16384, n_in, n_out, deg, peaks, alpha=0.5, beta=-0.3)
            sub["cfg3_shape_hermite_fp32"] = sub_family(ctx, "hermite", 16384, n_in, n_out, deg, peaks)
            for name in ("cfg1", "cfg2"):
                sub[name + "_train_eager"] = sub_small_train(ctx, name, False, 50, 5)
                sub[name + "_train_graph"] = sub_small_train(ctx, name, True, 200, 5)
            sub["cfg1_train_fused_step"] = sub_small_train(ctx, "cfg1", False, 200, 5, fused=True)

    if ctx.rank == 0:
        flops = 2.0 * B * n_in * (deg + 1) * n_out            # per GPU
        achieved = flops / (ms_step * 1e-3) / 1e12
        peak, peak_note = tensor_peak(mode, args.op, peaks, tf32_peak, n_out)
        traffic = measured_traffic(f"{args.op}_{mode}_cfg3", B) if not (args.shape or args.family) else None
        cfg = headline_config(ctx.world)
        if single:
            cfg = dict(cfg, workload=f"{args.family or 'chebyshev'} layer {args.op}, {Bg} rows x {n_in} -> {n_out}, degree {deg} (profiling run)",
                       global_batch=Bg, input_dim=n_in, output_dim=n_out, degree=deg)
        line = {
            "metric": METRIC if args.op == "fwd" else f"chebykan_layer_{args.op}_samples_per_s", "value": value,
            "unit": UNIT, "n_gpus": ctx.world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": DTYPE_NAME[mode], "data": "synthetic", "config": cfg,
            "arm": {"math_mode": mode, "op": args.op, "rows_per_gpu": B, "l2_flushed_between_steps": flushed},
            "roofline": {"bound": "tensor" if mode != "fp32" else "ffma", "achieved": achieved, "peak": peak,
                         "unit": "TFLOP/s", "frac": achieved / peak,
                         "traffic": traffic["bytes"] if traffic else None, "traffic_source": traffic,
                         "algorithmic_bytes": B * 4.0 * (n_in + n_out) + n_in * n_out * (deg + 1) * (2 if mode == "bf16" else 4),
                         "peak_note": peak_note, "flops_per_launch": flops, "per": "GPU",
                         "flops_executed": flops if mode == "fp32" else flops * deg / (deg + 1),
                         "flops_note": "achieved and frac count the layer's algorithmic FLOPs 2*B*in*(deg+1)*out; the "
                                       "tensor-core kernels execute deg/(deg+1) of them (plus one K block per tile): "
                                       "degree 0 of the basis is the constant 1, so its term sum_i C[i,o,0] is a bias "
                                       "vector, multiplied by a K block of ones (wide layers) or added in the "
                                       "epilogue (narrow layers)"},
            "e2e": e2e if e2e else {"value": None, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": args.steps,
            "clocks": clocks,
        }
        if tf32_peak:
            line["tf32_peak"] = tf32_peak
        if sub:
            line["sub"] = sub
        if ctx.world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline_cfg3() if not single else None
        print(json.dumps(line))
    ctx.close()


def run_model_config(args):
    """`--config cfgN`: one configuration's model step on its own (profiling and launch lists)."""
    ctx = Ctx()
    peaks = measured_peaks()
    from kan_b200 import workloads
    cfg = workloads.CONFIGS[args.config]
    if args.config == "cfg4":
        rec = sub_stack_cfg4(ctx, args.mode, args.fuse_ln, args.steps, args.warmup, peaks, None, batch=args.batch)
    elif args.config == "cfg5":
        rec = sub_train_cfg5(ctx, args.mode, args.steps, args.warmup, peaks, None, batch=args.batch,
                             torch_loss=args.torch_loss, graph=args.graph and not args.torch_loss)
    else:
        rec = sub_small_train(ctx, args.config, args.graph, args.steps, args.warmup)
    if ctx.rank == 0:
        line = {"metric": "chebykan_%s_samples_per_s" % ("train_step" if cfg.task == "train" else "stack_fwd"),
                "n_gpus": ctx.world, "steps": args.steps, "warmup": max(args.warmup, 3), "higher_is_better": True,
                "vs_baseline": None, "data": "synthetic", "config": {"workload": rec.get("workload", args.config)}}
        line.update(rec)
        if ctx.world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_model_baseline(cfg)
        print(json.dumps(line))
    ctx.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--mode", default="bf16", choices=["bf16", "tf32", "fp32", "fp32x3"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end leg (profiling runs)")
    ap.add_argument("--no-sub", action="store_true", help="headline only: skip the sub-records of the other configurations")
    ap.add_argument("--batch", type=int, default=0, help="global rows (default: the configuration's batch); profiling runs")
    ap.add_argument("--fuse-ln", action="store_true",
                    help="--config cfg4: fold the LayerNorms between layers into the ChebyKAN kernels")
    ap.add_argument("--graph", action="store_true",
                    help="--config cfg1/cfg2/cfg5: replay the whole step as one CUDA graph (cfg5: all-reduce included)")
    ap.add_argument("--torch-loss", action="store_true", help="--config cfg5: torch.nn.MSELoss instead of the fused loss")
    ap.add_argument("--op", default="fwd", choices=["fwd", "dcoeff", "dx"],
                    help="time the forward (headline) or one backward kernel on the same shape")
    ap.add_argument("--family", default="", choices=["", "jacobi", "hermite", "hermite_prob"],
                    help="profiling runs: the layer kernel with this polynomial family's recurrence (Jacobi alpha 0.5, beta -0.3)")
    ap.add_argument("--shape", default="", help="B,in,out,deg override (profiling other layer shapes)")
    ap.add_argument("--config", default="cfg3", choices=["cfg1", "cfg2", "cfg3", "cfg4", "cfg5"],
                    help="cfg3 (default) is the headline forward; the others time that configuration's model step alone")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.config != "cfg3":
        run_model_config(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
