"""Turn an ``ncu --page raw --csv`` export of one of this library's kernels into a short text summary and a
record in ``profiles/traffic.json`` (the measured DRAM bytes per launch that ``bench.py`` reports as
``roofline.traffic``).

    ncu -i capture.ncu-rep --page raw --csv > capture.csv
    python -m kan_b200.ncu_summary capture.csv --key fwd_tc_bf16_cfg3 --rows 32768 --fixed-bytes 18874368

``--rows`` is the batch the capture ran on and ``--fixed-bytes`` the part of the traffic that does not grow with
the batch (the packed coefficients); ``bench.py`` scales the rest to the rows of a full launch.  Without ``--key``
only the summary is printed.
"""
from __future__ import annotations

import argparse
import csv
import json
import os

WANT = [
    "gpu__time_duration.sum", "dram__bytes_read.sum", "dram__bytes_write.sum",
    "sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_active",
    "sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_elapsed",
    "gpu__dram_throughput.avg.pct_of_peak_sustained_elapsed", "lts__throughput.avg.pct_of_peak_sustained_elapsed",
    "lts__t_sector_hit_rate.pct", "smsp__issue_active.avg.pct_of_peak_sustained_active",
    "sm__inst_executed_pipe_fma.avg.pct_of_peak_sustained_active",
    "sm__inst_executed_pipe_alu.avg.pct_of_peak_sustained_active",
    "sm__inst_executed_pipe_xu.avg.pct_of_peak_sustained_active",
    "sm__inst_executed_pipe_lsu.avg.pct_of_peak_sustained_active", "smsp__inst_executed.sum",
    "sm__cycles_elapsed.avg.per_second", "l1tex__data_pipe_lsu_wavefronts_mem_shared.sum",
    "l1tex__data_bank_conflicts_pipe_lsu_mem_shared.sum", "launch__registers_per_thread", "launch__grid_size",
    "launch__block_size", "launch__shared_mem_per_block_dynamic", "sm__warps_active.avg.pct_of_peak_sustained_active",
    "smsp__pcsamp_warps_issue_stalled_long_scoreboard", "smsp__pcsamp_warps_issue_stalled_wait",
    "smsp__pcsamp_warps_issue_stalled_selected", "smsp__pcsamp_warps_issue_stalled_short_scoreboard",
    "smsp__pcsamp_warps_issue_stalled_math_pipe_throttle", "smsp__pcsamp_warps_issue_stalled_branch_resolving",
    "smsp__pcsamp_warps_issue_stalled_mio_throttle", "smsp__pcsamp_warps_issue_stalled_barrier",
    "smsp__pcsamp_warps_issue_stalled_not_selected", "smsp__pcsamp_warps_issue_stalled_dispatch_stall",
]

_SCALE = {"byte": 1.0, "Kbyte": 1e3, "Mbyte": 1e6, "Gbyte": 1e9, "ns": 1e-3, "us": 1.0, "ms": 1e3, "s": 1e6}


def read_capture(path: str):
    rows = list(csv.reader(open(path)))
    start = next(i for i, r in enumerate(rows) if r and r[0] == "ID")
    return rows[start], rows[start + 1], rows[start + 2:]


def column(hdr, units, launches, name):
    """Values of one metric over the captured launches, bytes in bytes and durations in microseconds."""
    if name not in hdr:
        return None
    i = hdr.index(name)
    scale = _SCALE.get(units[i], 1.0)
    out = []
    for r in launches:
        try:
            out.append(float(r[i].replace(",", "")) * scale)
        except ValueError:
            out.append(None)
    return out


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("csv")
    ap.add_argument("--key", default="", help="record name in profiles/traffic.json")
    ap.add_argument("--rows", type=int, default=0, help="batch rows of the captured launch")
    ap.add_argument("--fixed-bytes", type=float, default=0.0, help="traffic that does not scale with the rows")
    ap.add_argument("--command", default="", help="the capture command, stored with the record")
    ap.add_argument("--out", default=os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))),
                                                  "profiles", "traffic.json"))
    args = ap.parse_args()
    hdr, units, launches = read_capture(args.csv)
    ki = hdr.index("Kernel Name")
    for r in launches:
        print("kernel:", r[ki][:110])
    for name in WANT:
        vals = column(hdr, units, launches, name)
        if vals is not None:
            print(f"{name}: " + ", ".join("-" if v is None else f"{v:.6g}" for v in vals))
    if not args.key:
        return
    rd = column(hdr, units, launches, "dram__bytes_read.sum")
    wr = column(hdr, units, launches, "dram__bytes_write.sum")
    dur = column(hdr, units, launches, "gpu__time_duration.sum")
    if not rd or not wr or args.rows <= 0:
        raise SystemExit("the capture holds no dram__bytes_* columns, or --rows is missing")
    total = [a + b for a, b in zip(rd, wr)]
    rec = {"kernel": launches[0][ki][:110], "rows_captured": args.rows, "launches_captured": len(launches),
           "dram_bytes_per_launch": sum(total) / len(total), "dram_bytes_read": sum(rd) / len(rd),
           "dram_bytes_written": sum(wr) / len(wr), "fixed_bytes": args.fixed_bytes,
           "duration_us_under_ncu": (sum(dur) / len(dur)) if dur else None, "command": args.command}
    data = {}
    if os.path.exists(args.out):
        with open(args.out) as f:
            data = json.load(f)
    data[args.key] = rec
    with open(args.out, "w") as f:
        json.dump(data, f, indent=1, sort_keys=True)
        f.write("\n")
    print(f"wrote {args.key} -> {args.out}")


if __name__ == "__main__":
    main()
