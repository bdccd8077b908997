#!/usr/bin/env python3
"""Real-weights workflow: time the joint-sparse GEMM against cuBLAS on stored weight matrices.

Covers what the reference does with scripts/benchmark_real_weights.py (one weight tensor as B, a
dense synthetic A of 4096 rows, :186-264) and scripts/benchmark_ab_real.py (every compatible A x B
pair of two directories, :98-123, 223-311), with the same CSV columns, so the reference's plotting
and summary code reads the files unchanged.  What is different:

* no sudo, no profiler, no temporary .bin files and no child process: the matrices go to the GPU
  once and the library is called in this process; "compute" and "preprocess" are CUDA-event times
  of the GEMM launch and of the A pattern + packing launch (the reference sums profiler durations
  of kernels whose names contain "preprocess", scripts/benchmark.py:456-458);
* B's pattern bytes are computed once per weight file and kept beside it as <file>.bpat
  ("B offline, A per call", README.md:46,103); a cache written for another shape is recomputed;
* the K limit is the library's (65528), not 8192 (scripts/benchmark_real_weights.py:205-209).

Weight files: torch tensors (*.pt, 2-D, the reference's `*_permuted.pt` naming), NumPy arrays
(*.npy) or raw FP32 (*.bin with the shape in the name: <anything>_<rows>x<cols>.bin).

  python esmm-research_b200/real_weights.py --weights DIR [--kernels 15,29] [--rows 4096] [--out CSV]
  python esmm-research_b200/real_weights.py --weights-a DIR --weights-b DIR [--filter-a S] [--filter-b S]
"""
from __future__ import annotations

import argparse
import csv
import importlib.util
import os
import re
import sys
from pathlib import Path

import numpy as np

BM = 32          # rows of A (columns of B) per pattern byte
BK = 8           # K offsets per pattern byte
MAX_K = 65528    # the packed kernel lists k rows with 16-bit indices
JOINT_IDS = (20, 21, 25, 26, 27, 28, 29, 30)
A_TILE = {20: 64, 25: 64, 21: 8}


# ---- host-side helpers (no GPU, no library) ---------------------------------------------------
def pad_to_tile(arr: np.ndarray, row_tile: int = BM, col_tile: int = BK) -> np.ndarray:
    """Zero-pad to whole (row_tile x col_tile) tiles; the array itself when nothing is missing
    (scripts/benchmark_ab_real.py:36-44).  Zero padding adds only dead pattern bits."""
    rows, cols = arr.shape
    r = -(-rows // row_tile) * row_tile
    c = -(-cols // col_tile) * col_tile
    if (r, c) == (rows, cols):
        return arr
    out = np.zeros((r, c), dtype=arr.dtype)
    out[:rows, :cols] = arr
    return out


def compute_block_sparsity(arr: np.ndarray) -> float:
    """Fraction of all-zero 32 x 8 tiles (scripts/benchmark_ab_real.py:47-51); arr is tile-padded."""
    rows, cols = arr.shape
    tiles = arr.reshape(rows // BM, BM, cols // BK, BK)
    return float((np.abs(tiles).max(axis=(1, 3)) == 0).mean())


def parse_config(path: Path) -> dict:
    """Pruner, group size, permutation type and sparsity from the directory names of the reference's
    weight tree (scripts/benchmark_ab_real.py:54-70)."""
    cfg = {"pruner": "", "group_size": "", "perm_type": "", "sparsity": ""}
    for part in Path(path).parts:
        if part in ("wanda", "sparsegpt"):
            cfg["pruner"] = part
        if "grp_8" in part:
            cfg["group_size"] = "8"
        elif "grp_16" in part:
            cfg["group_size"] = "16"
        if "col_perm" in part or "columns_permuted" in part:
            cfg["perm_type"] = "col"
        elif "row_perm" in part or "rows_permuted" in part:
            cfg["perm_type"] = "row"
        if "sparsity_" in part:
            cfg["sparsity"] = part.split("sparsity_")[1].rstrip("/")
    return cfg


_BIN_SHAPE = re.compile(r"_(\d+)x(\d+)\.bin$")


def matrix_shape(path: Path):
    """Shape of a stored 2-D matrix, or None with a reason."""
    path = Path(path)
    try:
        if path.suffix == ".npy":
            arr = np.load(path, mmap_mode="r")
            return (tuple(arr.shape), None) if arr.ndim == 2 else (None, "not a 2D array")
        if path.suffix == ".bin":
            m = _BIN_SHAPE.search(path.name)
            if not m:
                return None, "no _<rows>x<cols> in the file name"
            shape = (int(m.group(1)), int(m.group(2)))
            if path.stat().st_size != 4 * shape[0] * shape[1]:
                return None, "file size does not match the shape in its name"
            return shape, None
        import torch
        obj = torch.load(path, map_location="cpu", weights_only=True)
        if not isinstance(obj, torch.Tensor) or obj.dim() != 2:
            return None, "not a 2D tensor"
        return tuple(obj.shape), None
    except Exception as e:  # unreadable file: skipped with the reason, like the reference
        return None, str(e)


def load_matrix(path: Path) -> np.ndarray:
    path = Path(path)
    if path.suffix == ".npy":
        return np.ascontiguousarray(np.load(path), dtype=np.float32)
    if path.suffix == ".bin":
        shape, why = matrix_shape(path)
        if shape is None:
            raise ValueError(f"{path}: {why}")
        return np.fromfile(path, dtype=np.float32).reshape(shape)
    import torch
    return torch.load(path, map_location="cpu", weights_only=True).float().contiguous().numpy()


def find_weight_files(root: Path, needle: str | None = None) -> list[Path]:
    root = Path(root)
    files = sorted(set(root.rglob("*_permuted.pt")) | set(root.rglob("*.npy")) | set(root.rglob("*x*.bin")))
    return [p for p in files if needle is None or needle in p.name]


def find_compatible_pairs(a_files, b_files, max_k: int = MAX_K, log=print) -> list:
    """(a, b) for every A whose column count equals B's row count, K within the limit, a != b
    (scripts/benchmark_ab_real.py:90-123)."""
    b_shapes = {}
    for b in b_files:
        shape, why = matrix_shape(b)
        if shape is None:
            log(f"  [SKIP B] {Path(b).name}: {why}")
            continue
        b_shapes[b] = shape
    pairs = []
    for a in a_files:
        shape, _ = matrix_shape(a)
        if shape is None:
            continue
        if shape[1] > max_k:
            log(f"  [SKIP A] {Path(a).name}: K={shape[1]} > {max_k}")
            continue
        pairs += [(a, b) for b, bs in b_shapes.items() if a != b and bs[0] == shape[1]]
    return pairs


def speedup_columns(row: dict, timings: dict) -> None:
    """k29_compute_speedup / k29_total_speedup against cuBLAS (scripts/benchmark_ab_real.py:296-306)."""
    if 15 in timings and 29 in timings:
        c15, _ = timings[15]
        c29, p29 = timings[29]
        if c15 and c29:
            row["k29_compute_speedup"] = f"{c15 / c29:.3f}"
            row["k29_total_speedup"] = f"{c15 / (c29 + (p29 or 0.0)):.3f}"
        else:
            row["k29_compute_speedup"] = row["k29_total_speedup"] = "N/A"


def timing_columns(row: dict, kernels, timings: dict) -> None:
    for k in kernels:
        c, p = timings.get(k, (None, None))
        row[f"k{k}_compute_ms"] = f"{c:.3f}" if c is not None else "N/A"
        row[f"k{k}_preprocess_ms"] = f"{p:.3f}" if p is not None else "N/A"


def write_csv(path: Path, rows: list[dict]) -> None:
    """Rewritten after every matrix so that partial results survive (scripts/benchmark_real_weights.py:301-305)."""
    path = Path(path)
    path.parent.mkdir(parents=True, exist_ok=True)
    with open(path, "w", newline="") as f:
        w = csv.DictWriter(f, fieldnames=list(rows[0].keys()))
        w.writeheader()
        w.writerows(rows)


def summary_lines(rows: list[dict]) -> list[str]:
    cs, ts = [], []
    for r in rows:
        try:
            cs.append(float(r["k29_compute_speedup"]))
            ts.append(float(r["k29_total_speedup"]))
        except (KeyError, ValueError):
            pass
    if not cs:
        return []
    return [f"K29 vs cuBLAS - {len(cs)} rows (CUDA-event timing):",
            f"  Compute-only: min={min(cs):.2f}x  max={max(cs):.2f}x  mean={sum(cs) / len(cs):.2f}x",
            f"  Total (incl. preprocess): min={min(ts):.2f}x  max={max(ts):.2f}x  mean={sum(ts) / len(ts):.2f}x"]


# ---- GPU side ---------------------------------------------------------------------------------------
def _package():
    """This package under an importable name (its directory name has a hyphen)."""
    name = "esmm_research_b200"
    if name in sys.modules:
        return sys.modules[name]
    here = Path(__file__).resolve().parent
    spec = importlib.util.spec_from_file_location(name, here / "__init__.py", submodule_search_locations=[str(here)])
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


class PairTimer:
    """One B (K x N) resident on the GPU with its cached pattern bytes; times kernel ids on A's."""

    def __init__(self, B: np.ndarray, cache_path: Path | None = None, log=print):
        import torch
        self.torch, self.pkg, self.L = torch, _package(), _package().lib()
        self.K, self.N = B.shape
        self.dB = torch.from_numpy(np.ascontiguousarray(B, dtype=np.float32)).cuda()
        nb = self.L.esmm_b_pattern_bytes(self.K, self.N)
        host = np.empty(nb, np.uint8)
        self.cache_state = "none"
        loaded = False
        if cache_path is not None and os.path.exists(cache_path):
            st = self.L.esmm_bpat_load(str(cache_path).encode(), host.ctypes.data, self.K, self.N)
            loaded = st == self.pkg.OK
            self.cache_state = "loaded" if loaded else "stale"
        if loaded:
            self.d_bpat = torch.from_numpy(host).cuda()
        else:
            self.d_bpat = torch.empty(nb, dtype=torch.uint8, device="cuda")
            self.pkg.preprocess_b(self.dB.data_ptr(), self.K, self.N, self.d_bpat.data_ptr())
            torch.cuda.synchronize()
            if cache_path is not None:
                host = self.d_bpat.cpu().numpy()
                st = self.L.esmm_bpat_save(str(cache_path).encode(), host.ctypes.data, self.K, self.N)
                self.cache_state = ("recomputed" if self.cache_state == "stale" else "saved") if st == self.pkg.OK \
                    else "unwritable"
        log(f"  B patterns: {self.cache_state}" + (f" ({cache_path})" if cache_path else ""))

    def _time(self, fn, runs: int, warmup: int = 2) -> float:
        t = self.torch
        for _ in range(warmup):
            fn()
        e0, e1 = t.cuda.Event(enable_timing=True), t.cuda.Event(enable_timing=True)
        t.cuda.synchronize()
        e0.record()
        for _ in range(runs):
            fn()
        e1.record()
        t.cuda.synchronize()
        return e0.elapsed_time(e1) / runs

    def time_kernels(self, A: np.ndarray, kernels, runs: int = 10, check: bool = True) -> dict:
        """{id: (compute_ms, preprocess_ms)}; (None, None) where an id failed or is unknown."""
        t, pkg = self.torch, self.pkg
        M, K = A.shape
        assert K == self.K
        dA = t.from_numpy(np.ascontiguousarray(A, dtype=np.float32)).cuda()
        dC = t.empty((M, self.N), dtype=t.float32, device="cuda")
        pA, pB, pC, pbp = dA.data_ptr(), self.dB.data_ptr(), dC.data_ptr(), self.d_bpat.data_ptr()
        out, ref = {}, None
        for kid in kernels:
            try:
                if kid == 15:
                    ms = self._time(lambda: pkg.cublas_sgemm(M, self.N, K, pA, pB, pC), runs)
                    out[kid] = (ms, 0.0)
                    ref = dC.clone()
                    continue
                if kid == 129:
                    # optional tensor-core variant: B prepared once per weight matrix (kept with this timer), the call
                    # does its own preprocessing of A, so the whole call is the "compute" column
                    if getattr(self, "tf32_b", None) is None:
                        self.tf32_b = pkg.Tf32x3B(pB, K, self.N, True)
                    ws = t.empty(pkg.tf32x3_workspace_bytes(M, K), dtype=t.uint8, device="cuda")
                    ms = self._time(lambda: pkg.sgemm_joint_tf32x3(M, pA, self.tf32_b, pC, ws.data_ptr()), runs)
                    pkg.device_status()
                    if check and ref is not None:
                        err = float((dC - ref).abs().max()) / max(float(ref.abs().max()), 1e-30)
                        if err > 1e-4:
                            raise pkg.EsmmError(pkg.ERR_VERIFY, f"kernel {kid}: rel-inf error {err:.3g} against cuBLAS")
                    out[kid] = (ms, 0.0)
                    continue
                if kid not in JOINT_IDS:
                    raise pkg.EsmmError(pkg.ERR_UNSUPPORTED, f"kernel id {kid}")
                tile = A_TILE.get(kid, 32)
                apat = t.empty(int(self.L.esmm_a_pattern_bytes(M, K, tile)), dtype=t.uint8, device="cuda")
                if tile == 32:
                    packed = t.empty(pkg.a_packed_bytes(M, K) // 4, dtype=t.float32, device="cuda")
                    pre = lambda: pkg.preprocess_a_packed(pA, M, K, apat.data_ptr(), packed.data_ptr())
                    run = lambda: pkg.gemm_ab_packed(M, self.N, K, packed.data_ptr(), pB, pC, apat.data_ptr(), pbp)
                else:
                    pre = lambda: pkg.preprocess_a(pA, M, K, apat.data_ptr(), tile)
                    run = lambda: pkg.gemm_ab(M, self.N, K, pA, pB, pC, apat.data_ptr(), pbp, tile)
                pre_ms = self._time(pre, runs)
                run_ms = self._time(run, runs)
                pkg.device_status()
                if check and ref is not None:
                    err = float((dC - ref).abs().max()) / max(float(ref.abs().max()), 1e-30)
                    if err > 1e-4:
                        raise pkg.EsmmError(pkg.ERR_VERIFY, f"kernel {kid}: rel-inf error {err:.3g} against cuBLAS")
                out[kid] = (run_ms, pre_ms)
            except pkg.EsmmError as e:
                print(f"    [ERROR] kernel={kid}: {e}")
                out[kid] = (None, None)
        return out


def _report(kernels, timings) -> None:
    for k in kernels:
        c, p = timings[k]
        label = "cuBLAS" if k == 15 else f"K{k}"
        print(f"  {label}: " + (f"compute={c:.3f}ms  preprocess={p:.3f}ms  total={c + p:.3f}ms" if c is not None else "FAILED"))


def benchmark_tensor(path: Path, kernels, rows: int = 4096, runs: int = 10, seed: int = 0, cache: bool = True):
    """One stored weight as B (K x N); A = rows x K of N(0,1), dense (scripts/benchmark_real_weights.py:186-264)."""
    shape, why = matrix_shape(path)
    if shape is None:
        print(f"  [SKIP] {Path(path).name}: {why}")
        return None
    W = load_matrix(path)
    B = pad_to_tile(W, BK, BM)
    if B.shape[0] > MAX_K:
        print(f"  [SKIP] K dimension {B.shape[0]} > {MAX_K}")
        return None
    cfg = parse_config(path)
    elem_sp = float((W == 0).mean())
    block_sp = compute_block_sparsity(pad_to_tile(W))
    print(f"\n{cfg['pruner']}/grp{cfg['group_size']}/{cfg['perm_type']}/sp{cfg['sparsity']}/{Path(path).stem[:35]}")
    print(f"  shape={shape}  elem={elem_sp * 100:.1f}%  block={block_sp * 100:.1f}%")
    timer = PairTimer(B, Path(str(path) + ".bpat") if cache else None)
    A = np.random.default_rng(seed).standard_normal((rows, B.shape[0]), dtype=np.float32)
    timings = timer.time_kernels(A, kernels, runs)
    _report(kernels, timings)
    row = {"layer": Path(path).stem, "pruner": cfg["pruner"], "group_size": cfg["group_size"],
           "perm_type": cfg["perm_type"], "sparsity": cfg["sparsity"], "orig_shape": f"{shape[0]}x{shape[1]}",
           "elem_sparsity_pct": f"{elem_sp * 100:.1f}", "block_sparsity_pct": f"{block_sp * 100:.1f}"}
    timing_columns(row, kernels, timings)
    speedup_columns(row, timings)
    return row


def benchmark_pair(a_path: Path, b_path: Path, kernels, runs: int = 10, cache: bool = True):
    """One stored A (M x K) times one stored B (K x N) (scripts/benchmark_ab_real.py:223-311)."""
    A0, B0 = load_matrix(a_path), load_matrix(b_path)
    A, B = pad_to_tile(A0, BM, BK), pad_to_tile(B0, BK, BM)
    a_cfg, b_cfg = parse_config(a_path), parse_config(b_path)
    a_block, b_block = compute_block_sparsity(A), compute_block_sparsity(pad_to_tile(B0))
    print(f"\n{Path(a_path).stem[:35]} x {Path(b_path).stem[:35]}")
    print(f"  A: shape={A0.shape}  elem={(A0 == 0).mean() * 100:.1f}%  block={a_block * 100:.1f}%")
    print(f"  B: shape={B0.shape}  elem={(B0 == 0).mean() * 100:.1f}%  block={b_block * 100:.1f}%")
    timer = PairTimer(B, Path(str(b_path) + ".bpat") if cache else None)
    timings = timer.time_kernels(A, kernels, runs)
    _report(kernels, timings)
    row = {"a_file": Path(a_path).stem, "b_file": Path(b_path).stem, "a_pruner": a_cfg["pruner"],
           "b_pruner": b_cfg["pruner"], "a_sparsity": a_cfg["sparsity"], "b_sparsity": b_cfg["sparsity"],
           "a_block_sparsity_pct": f"{a_block * 100:.1f}", "b_block_sparsity_pct": f"{b_block * 100:.1f}",
           "a_shape": f"{A0.shape[0]}x{A0.shape[1]}", "b_shape": f"{B0.shape[0]}x{B0.shape[1]}"}
    timing_columns(row, kernels, timings)
    speedup_columns(row, timings)
    return row


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="Joint-sparse GEMM vs cuBLAS on stored weight matrices.")
    ap.add_argument("--weights", help="directory of weight files used as B; A is dense synthetic")
    ap.add_argument("--weights-a", help="directory of weight files used as A")
    ap.add_argument("--weights-b", help="directory of weight files used as B")
    ap.add_argument("--filter-a", default=None, help="only A files whose name contains this")
    ap.add_argument("--filter-b", default=None, help="only B (or --weights) files whose name contains this")
    ap.add_argument("--kernels", default="15,29", help="comma-separated kernel ids (default 15,29)")
    ap.add_argument("--rows", type=int, default=4096, help="rows of the synthetic A in --weights mode")
    ap.add_argument("--runs", type=int, default=10)
    ap.add_argument("--no-cache", action="store_true", help="do not read or write <file>.bpat")
    ap.add_argument("--out", default=None, help="CSV path")
    args = ap.parse_args(argv)
    kernels = [int(k) for k in args.kernels.split(",")]
    pair_mode = bool(args.weights_a or args.weights_b)
    if pair_mode == bool(args.weights) or (pair_mode and not (args.weights_a and args.weights_b)):
        ap.error("give either --weights, or both --weights-a and --weights-b")
    _package().lib()  # fails here, loudly, when the library has not been built

    rows_out = []
    if not pair_mode:
        out = Path(args.out or "results/real_weights_benchmark.csv")
        files = find_weight_files(args.weights, args.filter_b)
        if not files:
            print(f"No weight files found in {args.weights}")
            return 1
        print(f"Found {len(files)} weight matrices | kernels={kernels} | timing=CUDA events")
        for f in files:
            row = benchmark_tensor(f, kernels, args.rows, args.runs, cache=not args.no_cache)
            if row:
                rows_out.append(row)
                write_csv(out, rows_out)
    else:
        out = Path(args.out or "results/ab_real_benchmark.csv")
        a_files = find_weight_files(args.weights_a, args.filter_a)
        b_files = find_weight_files(args.weights_b, args.filter_b)
        if not a_files or not b_files:
            print(f"No {'A' if not a_files else 'B'} files found")
            return 1
        pairs = find_compatible_pairs(a_files, b_files)
        if not pairs:
            print("No compatible A x B pairs found (check shapes and K limit).")
            return 1
        print(f"A files: {len(a_files)} | B files: {len(b_files)} | Compatible pairs: {len(pairs)} | kernels={kernels}")
        for a, b in pairs:
            row = benchmark_pair(a, b, kernels, args.runs, cache=not args.no_cache)
            if row:
                rows_out.append(row)
                write_csv(out, rows_out)
    for line in summary_lines(rows_out):
        print(line)
    print(f"\nResults saved to {out}  ({len(rows_out)} rows)")
    return 0


if __name__ == "__main__":
    sys.exit(main())
