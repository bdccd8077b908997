#!/usr/bin/env python3
"""Size x pattern sweep of kernel ids through the driver CLI, one CSV row per run.

Covers what the reference's scripts/benchmark.py does (defaults :27-33: sizes 1024, 2048, 4096 and
the patterns 11111111 / 11110000 / 11000000 / 10000000; options :49-135), without a profiler: each
point is one `exec_b200 <kernels> <runs> ... --no-check --json` call and the times are the runner's own
CUDA-event averages ("Kernel time", include/runners.cuh:868-872), i.e. the reference-style loop with
its per-run memset, pattern allocation and preprocessing inside.  With --cusparse every point also
gets the cuSPARSE SpMM row of cusparse_bench at the pattern's density.

  python esmm-research_b200/sweep.py -k 29,15 [--sizes 1024,2048,4096] [--sparsity P,P,...]
         [-pa P -pb P] [--blockwise | --uniform] [--runs 10] [--cusparse] [--output results/sweep.csv]
"""
from __future__ import annotations

import argparse
import csv
import json
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
DEFAULT_SIZES = [1024, 2048, 4096]
DEFAULT_SPARSITY = {"100pct": "11111111", "50pct": "11110000", "25pct": "11000000", "12pct": "10000000"}
FIELDS = ["kernel", "size", "pattern_a", "pattern_b", "mode", "density_a", "density_b", "runs", "avg_ms",
          "dense_equiv_tflops", "status"]
SPARSE_FIELDS = ["size", "density", "spmm_us", "total_us", "spmm_gflops", "total_gflops", "esmm_us", "cublas_us",
                 "rel_diff"]


def valid_pattern(p: str) -> bool:
    return len(p) == 8 and set(p) <= {"0", "1"}


def density(p: str) -> float:
    return p.count("1") / 8.0


def plan_points(sizes, patterns, pattern_a=None, pattern_b=None):
    """(size, pattern for A, pattern for B) of every run; -pa / -pb replace the swept pattern for that operand
    (scripts/benchmark.py:67-78)."""
    pts = []
    for n in sizes:
        if pattern_a and pattern_b:
            pts.append((n, pattern_a, pattern_b))
            continue
        for p in patterns:
            pts.append((n, pattern_a or p, pattern_b or p))
    return pts


def driver_command(kernels: str, runs: int, size: int, pa: str, pb: str, mode: str) -> list[str]:
    cmd = [str(HERE / "exec_b200"), kernels, str(runs), "--size", str(size), "--pattern-a", pa, "--pattern-b", pb,
           "--no-check", "--json"]
    if mode == "blockwise":
        cmd.append("--blockwise")
    elif mode == "uniform":
        cmd.append("--uniform")
    return cmd


def parse_driver_output(text: str, size: int, pa: str, pb: str, mode: str) -> list[dict]:
    rows = []
    for line in text.splitlines():
        line = line.strip()
        if not (line.startswith("{") and '"kernel"' in line):
            continue
        d = json.loads(line)
        rows.append({"kernel": d["kernel"], "size": size, "pattern_a": pa, "pattern_b": pb, "mode": mode,
                     "density_a": density(pa), "density_b": density(pb), "runs": d["runs"],
                     "avg_ms": f"{d['avg_ms']:.4f}", "dense_equiv_tflops": f"{d['dense_equiv_tflops']:.2f}",
                     "status": d["status"]})
    return rows


def parse_sparse_row(text: str) -> dict | None:
    for line in text.splitlines():
        parts = line.strip().split(",")
        if len(parts) in (6, 9) and parts[0].isdigit():
            return dict(zip(SPARSE_FIELDS, parts))
    return None


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="Sweep kernel ids over sizes and sparsity patterns")
    ap.add_argument("-k", "--kernel", required=True, help="kernel ids, the driver's grammar: 29 / 29,15 / 14-17 / all")
    ap.add_argument("-s", "--sizes", default=",".join(map(str, DEFAULT_SIZES)))
    ap.add_argument("-p", "--sparsity", default=None, help="comma-separated 8-bit patterns (default 100/50/25/12.5 %%)")
    ap.add_argument("-pa", "--pattern-a", default=None)
    ap.add_argument("-pb", "--pattern-b", default=None)
    ap.add_argument("-b", "--blockwise", action="store_true", help="the driver's --blockwise data (random per-tile patterns)")
    ap.add_argument("-u", "--uniform", action="store_true", help="the driver's --uniform data (N(0,1), pattern on A's K columns and B's K rows)")
    ap.add_argument("--runs", type=int, default=10)
    ap.add_argument("--cusparse", action="store_true", help="add cuSPARSE SpMM rows (cusparse_bench --compare)")
    ap.add_argument("-o", "--output", default="results/sweep.csv")
    args = ap.parse_args(argv)

    sizes = [int(x) for x in args.sizes.split(",") if x]
    patterns = args.sparsity.split(",") if args.sparsity else list(DEFAULT_SPARSITY.values())
    for p in patterns + [x for x in (args.pattern_a, args.pattern_b) if x]:
        if not valid_pattern(p):
            print(f"Error: pattern '{p}' must be 8 characters of 0 and 1")
            return 1
    if args.blockwise and args.uniform:
        print("Error: --blockwise and --uniform exclude each other")
        return 1
    mode = "blockwise" if args.blockwise else "uniform" if args.uniform else "column"
    if not (HERE / "exec_b200").exists():
        print(f"Error: {HERE / 'exec_b200'} not found: run `python esmm-research_b200/build.py`")
        return 1

    out = Path(args.output)
    out.parent.mkdir(parents=True, exist_ok=True)
    rows, sparse_rows = [], []
    for size, pa, pb in plan_points(sizes, patterns, args.pattern_a, args.pattern_b):
        cmd = driver_command(args.kernel, args.runs, size, pa, pb, mode)
        r = subprocess.run(cmd, capture_output=True, text=True)
        got = parse_driver_output(r.stdout, size, pa, pb, mode)
        if not got:
            print(f"[FAIL] size {size} A {pa} B {pb}: exit {r.returncode}\n{r.stdout[-400:]}{r.stderr[-400:]}")
            continue
        rows += got
        for g in got:
            print(f"size {size:6d}  A {pa} B {pb}  kernel {g['kernel']:3d}  {g['avg_ms']:>10s} ms  {g['dense_equiv_tflops']:>8s} TFLOP/s dense-equivalent")
        if args.cusparse:
            r = subprocess.run([str(HERE / "cusparse_bench"), "--size", str(size), "--density", str(density(pa)),
                                "--runs", str(args.runs), "--compare"], capture_output=True, text=True)
            s = parse_sparse_row(r.stdout)
            if s:
                sparse_rows.append(s)
                print(f"size {size:6d}  density {s['density']}  cuSPARSE spmm {s['spmm_us']} us, with conversion {s['total_us']} us")
        with open(out, "w", newline="") as f:   # rewritten after every point: partial results survive
            w = csv.DictWriter(f, fieldnames=FIELDS)
            w.writeheader()
            w.writerows(rows)
        if sparse_rows:
            with open(out.with_name(out.stem + "_cusparse.csv"), "w", newline="") as f:
                w = csv.DictWriter(f, fieldnames=SPARSE_FIELDS)
                w.writeheader()
                w.writerows(sparse_rows)
    print(f"\nResults saved to {out} ({len(rows)} rows)")
    return 0 if rows else 1


if __name__ == "__main__":
    sys.exit(main())
