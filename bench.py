#!/usr/bin/env python
"""Benchmark of the joint-sparse SGEMM hot path (A-pattern preprocess + GEMM) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c2|c5]

One JSON line on stdout (rank 0).  Metric: dense-equivalent TFLOP/s (2 M N K / t), including the
per-call A preprocessing, B patterns cached.

N = 1 (default): workload "c2" - M = N = K = 4096 FP32, N(0,1) inputs, uniform blockwise patterns
  11111111 / 11110000 / 11000000 / 10000000 (100 / 50 / 25 / 12.5 % joint density) applied to A's K
  columns and B's K rows.  One step = the four densities once, each = packing preprocess of A +
  GEMM.  `value` is the sweep's aggregate (4 * 2 * 4096^3 flops / step time); the per-density
  figures, cuBLAS SGEMM on the same inputs and the roofline fractions are in "sweep".
N > 1 (torchrun, one process per GPU): workload "c5" - M = N = K = 16384, pattern 11000000, B and
  C column-sharded over the ranks, A and its preprocessing replicated, no data-path collective.
  `value` = 2 * 16384^3 / (max over ranks of the device time); strong scaling.

--impl reference times the reference's own CPU SGEMM (matrixMultiplyCPU, compiled from the reference
tree into oracle/_ref, else the oracle's restatement of it) on all host cores over a bounded row
sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

PATTERNS = [("11111111", 0xFF), ("11110000", 0x0F), ("11000000", 0x03), ("10000000", 0x01)]
NOMINAL_FP32_TFLOPS = 148 * 128 * 2 * 1.965e9 / 1e12  # 74.4: 148 SMs x 128 lanes x 2 flop x max SM clock


def measured_peaks() -> dict:
    try:
        return json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        return {}


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons while the timed region runs: NVML queries (read-only) every 10 ms,
    or, where the NVML binding is unusable, nvidia-smi as fast as it answers."""

    REASONS = (("hw_slowdown", 0x8), ("hw_thermal_slowdown", 0x40), ("sw_thermal_slowdown", 0x20), ("sw_power_cap", 0x4))

    def __init__(self, index: int, uuid: str | None = None):
        super().__init__(daemon=True)
        self.index, self.uuid, self.stop_flag, self.rows, self.source = index, uuid, threading.Event(), [], "nvml"
        try:                                  # initialised here, outside the timed region (it takes tens of ms)
            self.nv, self.handle = self._nvml_handle()
            self.max_mhz = self.nv.nvmlDeviceGetMaxClockInfo(self.handle, self.nv.NVML_CLOCK_SM)
        except Exception:
            self.nv = self.handle = None

    def _nvml_handle(self):
        import pynvml
        pynvml.nvmlInit()
        if self.uuid:
            try:
                return pynvml, pynvml.nvmlDeviceGetHandleByUUID(self.uuid)
            except Exception:
                pass
        return pynvml, pynvml.nvmlDeviceGetHandleByIndex(self.index)

    def run(self):
        try:
            if self.nv is None:
                raise RuntimeError("no NVML")
            nv, h, mx = self.nv, self.handle, self.max_mhz
            while not self.stop_flag.is_set():
                sm = nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(h)
                self.rows.append((sm, mx, [n for n, bit in self.REASONS if mask & bit]))
                self.stop_flag.wait(0.01)
            return
        except Exception:
            self.source = "nvidia-smi"
        q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
        while not self.stop_flag.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--id={self.index}", f"--query-gpu={q}",
                                      "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=5).stdout
                parts = [p.strip() for p in out.strip().split(",")]
                if len(parts) >= 6 and parts[0].isdigit() and parts[1].isdigit():
                    self.rows.append((int(parts[0]), int(parts[1]),
                                      [n for (n, _), v in zip(self.REASONS, parts[2:6]) if v.lower().startswith("active")]))
            except Exception:
                pass
            self.stop_flag.wait(0.05)

    def summary(self) -> dict:
        self.stop_flag.set()
        self.join(timeout=6)
        sm = sorted(r[0] for r in self.rows)
        mx = [r[1] for r in self.rows]
        reasons = sorted({n for r in self.rows for n in r[2]})
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(self.rows), "source": self.source}


def host_threads() -> int:
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except Exception:
        return max(1, os.cpu_count() or 1)


# ---------------------------------------------------------------------------------------------------
# reference arm / CPU baseline: the reference's CPU SGEMM on a bounded row sample
# ---------------------------------------------------------------------------------------------------
class CpuSgemm:
    def __init__(self, M: int, N: int, K: int, pattern: int, seed: int = 0):
        import numpy as np
        import oracle
        self.oracle, self.np = oracle, np
        self.M, self.N, self.K = M, N, K
        self.threads = host_threads()
        self.kind = "reference" if oracle.have_ref() else "port"
        rng = np.random.default_rng(seed)
        live = np.array([(pattern >> (k & 7)) & 1 for k in range(K)], dtype=np.float32)
        self.B = rng.standard_normal((K, N), dtype=np.float32) * live[:, None]
        self.A_rows = None
        self.live = live
        self.rng = rng

    def run(self, rows: int) -> float:
        """Seconds for `rows` rows of C (all N columns), split over all host threads."""
        np = self.np
        if self.A_rows is None or self.A_rows.shape[0] != rows:
            self.A_rows = self.rng.standard_normal((rows, self.K), dtype=np.float32) * self.live[None, :]
        t0 = time.perf_counter()
        if self.kind == "reference":
            self.oracle.ref_sgemm_cpu(self.A_rows, self.B, threads=self.threads)
        else:
            self.oracle.sgemm_naive(self.A_rows, self.B, threads=self.threads)
        return time.perf_counter() - t0

    def calibrate(self, target_s: float) -> int:
        rows = self.threads
        dt = self.run(rows)
        per_row = max(dt / rows, 1e-6)
        want = int(target_s / per_row)
        want = max(self.threads, min(want, self.M))
        return (want // self.threads) * self.threads or self.threads


METRIC_C2 = "dense-equivalent TFLOP/s at 4096^3 FP32 vs block density, incl. A-pattern preprocess"
METRIC_C5 = "dense-equivalent TFLOP/s at 16384^3 FP32, 25% joint density, incl. A-pattern preprocess"


def run_reference_arm(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    if args.gpus > 1 or args.workload == "c5":
        M = N = K = 16384
        wl, pat = "c5: 16384^3 FP32, pattern 11000000 (25% joint density)", 0x03
    else:
        M = N = K = 4096
        wl, pat = "c2: 4096^3 FP32, uniform pattern sweep 100/50/25/12.5% (CPU SGEMM is dense: time is density independent)", 0xFF
    cpu = CpuSgemm(M, N, K, pat)
    rows = cpu.calibrate(target_s=2.0 if M <= 4096 else 4.0)
    for _ in range(args.warmup):
        cpu.run(rows)
    t = 0.0
    for _ in range(args.steps):
        t += cpu.run(rows)
    per_step = t / args.steps
    tflops = 2.0 * rows * N * K / per_step / 1e12
    sample = f"{rows} of {M} rows of C (all {N} columns, full K) per step; time scales linearly in rows"
    line = {
        "impl": "reference", "metric": METRIC_C5 if M > 4096 else METRIC_C2, "value": tflops,
        "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": per_step * 1e3, "higher_is_better": True, "scaling": "strong" if args.gpus > 1 else "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": wl, "M": M, "N": N, "K": K, "sample": sample},
        "cpu_baseline": {"value": tflops, "unit": "TFLOP/s", "cores": cpu.threads, "kind": cpu.kind, "sample": sample},
        "e2e": {"value": tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------------
# comparison columns and checks around the timed step (never inside it)
# ---------------------------------------------------------------------------------------------------
def ref_kernel_times(M, N, K, A, B, ours_ms, dev):
    """The reference's own GPU kernels (its pattern preprocessors and kernel id 29, compiled for sm_100a from the
    reference tree into oracle/_ref) timed with CUDA events on the same device buffers: a comparison column beside
    cuBLAS.  None when oracle/_ref is absent or the shape is outside the reference kernel's limits."""
    import torch
    try:
        import oracle
        if not oracle.have_ref() or M % 64 or N % 128 or K % 8 or K > 8192:
            return None
        ra = torch.empty((M // 32) * (K // 8), dtype=torch.uint8, device=dev)
        rb = torch.empty((N // 32) * (K // 8), dtype=torch.uint8, device=dev)
        Cr = torch.empty((M, N), device=dev)
        pre_a, pre_b, gemm = oracle.ref_time_kernels(M, N, K, A.data_ptr(), B.data_ptr(), Cr.data_ptr(), ra.data_ptr(),
                                                     rb.data_ptr(), warmup=2, runs=5)
        return {"ms_ref_pre_a": pre_a, "ms_ref_pre_b": pre_b, "ms_ref_pre": pre_a + pre_b, "ms_ref_id29": gemm,
                "speedup_vs_ref_b_offline": (pre_a + gemm) / ours_ms,       # both sides: A patterns per call, B cached
                "speedup_vs_ref_own_loop": (pre_a + pre_b + gemm) / ours_ms}  # the reference recomputes B every run
    except Exception as e:  # a comparison column must not break the bench line
        return {"error": str(e)[:200]}


def other_config_rows(pkg, torch, dev, time_each):
    """Configs 3 and 4 (not part of `value`): this library's per-call path, cuBLAS SGEMM and, where its shape limits
    allow, the reference's kernels, on the same inputs."""
    import numpy as np
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import workloads
    L = pkg.lib()
    rows = {}

    def measure(name, A, B):
        M, K = A.shape
        N = B.shape[1]
        bp = torch.empty(L.esmm_b_pattern_bytes(K, N), dtype=torch.uint8, device=dev)
        pkg.preprocess_b(B.data_ptr(), K, N, bp.data_ptr())
        ws = torch.empty(pkg.sgemm_joint_workspace_bytes(M, K), dtype=torch.uint8, device=dev)
        Cm = torch.empty((M, N), device=dev)
        ours, ours_min = time_each(lambda: pkg.sgemm_joint(M, N, K, A.data_ptr(), B.data_ptr(), Cm.data_ptr(),
                                                           bp.data_ptr(), ws.data_ptr()), 10)
        cub, _ = time_each(lambda: pkg.cublas_sgemm(M, N, K, A.data_ptr(), B.data_ptr(), Cm.data_ptr()), 10)
        nmb, nkb = -(-M // 32), -(-K // 8)
        ap = ws[:nmb * nkb].reshape(nmb, nkb).cpu().numpy()
        bpat = bp.reshape(-1, nkb).cpu().numpy()
        # executed multiply-adds = 32 * 32 * sum popcount(a & b) over (row block, column block, K block)
        bits_a = np.unpackbits(ap, axis=1).astype(np.float32).T         # [nkb * 8, nmb]
        bits_b = np.unpackbits(bpat, axis=1).astype(np.float32).T       # [nkb * 8, nnb]
        joint = float((bits_a.sum(axis=1) * bits_b.sum(axis=1)).sum()) / (bits_a.shape[1] * bits_b.shape[1] * nkb * 8)
        rows[name] = {"M": M, "N": N, "K": K, "joint_density": joint, "ms_total": ours, "ms_total_min": ours_min,
                      "ms_cublas": cub, "speedup_vs_cublas_incl_pre": cub / ours,
                      "dense_equiv_tflops_incl_pre": 2.0 * M * N * K / (ours * 1e-3) / 1e12,
                      "executed_tflops_incl_pre": 2.0 * M * N * K * joint / (ours * 1e-3) / 1e12,
                      "reference_kernels": ref_kernel_times(M, N, K, A, B, ours, dev)}

    S = 4096
    for pA, pB in ((0.5, 0.5), (0.3, 0.7), (0.2, 0.2)):
        A = torch.empty((S, S), device=dev)
        B = torch.empty((S, S), device=dev)
        pkg.fill_normal(A.data_ptr(), S, S, 0, 11, mode=2, p_live=pA, gran=64, seed2=101)
        pkg.fill_normal(B.data_ptr(), S, S, 1, 12, mode=2, p_live=pB, gran=64, seed2=102)
        measure(f"c3 pA={pA} pB={pB} (64-granular tile patterns)", A, B)
    for M4 in (2048, 16):
        hA, hB = workloads.llm_mlp(M4, 11008, 4096, seed=40 + M4)
        measure(f"c4 M={M4} K=4096 N=11008 (LLM MLP)", torch.from_numpy(hA).to(dev), torch.from_numpy(hB).to(dev))
    # The reference's own headline inputs (README: `exec 29,15 10 --blockwise --pattern P --size 4096`): an independent
    # random 8-bit pattern per 32 x 8 tile of A and 8 x 32 tile of B, bit density popcount(P) / 8, values {0..4} +
    # 0.01 {0..4} with a random sign, seeds 12345 / 12346 - drawn by the library's restatement of the driver's rand()
    # generators (bit for bit the reference's matrices).
    hA = np.zeros((S, S), np.float32)
    hB = np.zeros((S, S), np.float32)
    for pattern in ("11110000", "11000000", "10000000"):
        sparsity = 100.0 - pattern.count("1") / 8.0 * 100.0
        pkg.check(L.esmm_randomize_matrix_a_blocklevel(hA.ctypes.data, S, S, 8, 32, sparsity, 12345), "generator A")
        pkg.check(L.esmm_randomize_matrix_b_blocklevel(hB.ctypes.data, S, S, 8, 32, sparsity, 12346), "generator B")
        measure(f"reference README inputs: --blockwise --pattern {pattern} --size {S}", torch.from_numpy(hA).to(dev),
                torch.from_numpy(hB).to(dev))
    pkg.device_status()
    return rows


def check_shard_against_oracle(pkg, torch, A, B, Cd, blocks=3):
    """Untimed correctness check of one rank's column shard: pattern bytes of the B shard in full, and C on a few
    32-row blocks, against the CPU oracle (the checker, never the thing measured).  Returns a small dict."""
    import numpy as np
    import oracle
    M, K = A.shape
    Nl = B.shape[1]
    hB = B.cpu().numpy()
    obp = oracle.preprocess_b(hB)
    nb = M // 32
    picks = sorted({0, nb - 1} | {int(x) for x in np.linspace(0, nb - 1, blocks + 2)[1:-1]})
    worst, bits = 0.0, True
    for blk in picks:
        hA = A[blk * 32:(blk + 1) * 32].cpu().numpy()
        want = oracle.gemm_joint(hA, hB, oracle.preprocess_a(hA), obp)
        got = Cd[blk * 32:(blk + 1) * 32].cpu().numpy()
        worst = max(worst, oracle.rel_inf_err(got, want))
        bits = bits and bool(np.array_equal(got, want))
    return {"passed": bool(worst <= 1e-4), "bit_identical": bits, "max_rel_inf": worst, "rows_checked": 32 * len(picks),
            "columns": Nl, "row_blocks": picks}


# ---------------------------------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------------------------------
def run_ours(args) -> None:
    import numpy as np
    import torch
    import __graft_entry__ as g

    pkg = g.load_package()  # raises if the CUDA library is missing: there is no fallback
    L = pkg.lib()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the product path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    import importlib
    sharding = importlib.import_module("esmm_research_b200.sharding")

    workload = args.workload or ("c5" if world > 1 else "c2")
    peaks = measured_peaks()
    ffma_peak, sms = pkg.ffma_peak_tflops()
    hbm_peak = float(peaks.get("hbm_gbs", 6650.0))
    hbm_src = "measured" if "hbm_gbs" in peaks else "fallback"

    def ev():
        return torch.cuda.Event(enable_timing=True)

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- problem set-up (untimed) ----
    if workload == "c2":
        M = N = K = args.size or 4096
        pats = PATTERNS
        shard = sharding.shard_columns(N, world, rank) if world > 1 else sharding.ColumnShard(0, 1, N, 0, N)
    else:
        M = N = K = args.size or 16384
        pats = [("11000000", 0x03)]
        shard = sharding.shard_columns(N, world, rank)
    Nl = shard.width
    cases = []
    for name, pat in pats:
        A = torch.empty((M, K), device=dev)
        B = torch.empty((K, Nl), device=dev)
        pkg.fill_normal(A.data_ptr(), M, K, 0, 1, mode=1, pattern=pat)               # same A on every rank
        pkg.fill_normal(B.data_ptr(), K, Nl, 1, 1000 + rank, mode=1, pattern=pat)    # this rank's columns
        bp = torch.empty(L.esmm_b_pattern_bytes(K, Nl), dtype=torch.uint8, device=dev)
        pkg.preprocess_b(B.data_ptr(), K, Nl, bp.data_ptr())                         # offline: B patterns cached
        cases.append(dict(name=name, pat=pat, A=A, B=B, bp=bp))
    Cd = torch.empty((M, Nl), device=dev)
    ws = torch.empty(pkg.sgemm_joint_workspace_bytes(M, K), dtype=torch.uint8, device=dev)
    ap_bytes = int(L.esmm_a_pattern_bytes(M, K, 32))
    ap_region = (ap_bytes + 255) & ~255
    flops_dense = 2.0 * M * N * K           # whole job, per density
    flops_dense_local = 2.0 * M * Nl * K
    torch.cuda.synchronize()

    def step():
        for c in cases:
            pkg.sgemm_joint(M, Nl, K, c["A"].data_ptr(), c["B"].data_ptr(), Cd.data_ptr(), c["bp"].data_ptr(),
                            ws.data_ptr())

    # ---- timed region: W warm-up + K steps, device time, max over ranks ----
    for _ in range(max(args.warmup, 3)):
        step()
    pkg.device_status()
    shard_check = None
    if dist is not None and not args.no_check:
        # every rank checks its own shard (untimed); the line reports the result over all ranks
        mine = check_shard_against_oracle(pkg, torch, cases[0]["A"], cases[0]["B"], Cd)
        flags = torch.tensor([1 if mine["passed"] else 0, 1 if mine["bit_identical"] else 0], dtype=torch.int32, device=dev)
        dist.all_reduce(flags, op=dist.ReduceOp.MIN)
        shard_check = dict(mine, all_ranks_passed=bool(flags[0].item() == 1), all_ranks_bit_identical=bool(flags[1].item() == 1),
                           what="C of this rank's column shard on sampled 32-row blocks and the B pattern bytes in full "
                                "against the CPU oracle, before the timed region; flags all-reduced (MIN) over the ranks")
    try:
        gpu_uuid = "GPU-" + str(torch.cuda.get_device_properties(local_rank).uuid)
    except Exception:
        gpu_uuid = None
    sampler = ClockSampler(local_rank, gpu_uuid)
    if rank == 0:
        sampler.start()
    barrier()
    e0, e1 = ev(), ev()
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    pkg.device_status()
    ms_total = sharding.max_over_ranks(e0.elapsed_time(e1), dist, dev) if dist is not None else e0.elapsed_time(e1)
    clocks = sampler.summary() if rank == 0 else {}
    ms_step = ms_total / args.steps
    value = len(cases) * flops_dense / (ms_step * 1e-3) / 1e12

    # ---- per-kernel durations (separate loop, same stream) for the roofline and the sweep table ----
    def time_each(fn, reps):
        for _ in range(2):
            fn()
        ts = []
        for _ in range(reps):
            a, b = ev(), ev()
            a.record()
            fn()
            b.record()
            b.synchronize()
            ts.append(a.elapsed_time(b))
        return float(np.mean(ts)), float(np.min(ts))

    reps = max(5, min(20, args.steps))
    sweep = {}
    gemm_ms_sum = 0.0
    exec_flops_sum = 0.0
    pre_ms_sum = 0.0
    pack = ws[ap_region:]
    # The packing preprocess is a 20-30 us kernel at 4096^2: timed one launch at a time, launch latency and the
    # events themselves are a third of the figure.  So it is timed as a train of back-to-back launches over
    # rotating copies of A (3 x 67 MB, more than L2 holds) between one pair of events.
    def time_train(fn_of_index, launches):
        for i in range(3):
            fn_of_index(i)
        a, b = ev(), ev()
        a.record()
        for i in range(launches):
            fn_of_index(i)
        b.record()
        b.synchronize()
        return a.elapsed_time(b) / launches

    for c in cases:
        pre_single_ms, _ = time_each(lambda: pkg.preprocess_a_packed(c["A"].data_ptr(), M, K, ws.data_ptr(),
                                                                     pack.data_ptr()), reps)
        if 4.0 * M * K < 512e6:
            copies = [c["A"], c["A"].clone(), c["A"].clone()]
            pre_ms = time_train(lambda i: pkg.preprocess_a_packed(copies[i % 3].data_ptr(), M, K, ws.data_ptr(),
                                                                  pack.data_ptr()), 24)
            del copies
        else:
            pre_ms = pre_single_ms          # a large A: one launch is long enough and A alone exceeds L2
        pkg.preprocess_a_packed(c["A"].data_ptr(), M, K, ws.data_ptr(), pack.data_ptr())   # patterns of THIS case for the GEMM below
        gemm_ms, gemm_min = time_each(lambda: pkg.gemm_ab_packed(M, Nl, K, pack.data_ptr(), c["B"].data_ptr(),
                                                                 Cd.data_ptr(), ws.data_ptr(), c["bp"].data_ptr()), reps)
        both_ms, _ = time_each(lambda: pkg.sgemm_joint(M, Nl, K, c["A"].data_ptr(), c["B"].data_ptr(), Cd.data_ptr(),
                                                       c["bp"].data_ptr(), ws.data_ptr()), reps)
        cub_ms, _ = time_each(lambda: pkg.cublas_sgemm(M, Nl, K, c["A"].data_ptr(), c["B"].data_ptr(),
                                                       Cd.data_ptr()), reps)
        # optional tensor-core variant (3xTF32, inside the 1e-4 tolerance but not bit-identical): reported beside
        # the FP32 path, never part of `value`
        tb = pkg.Tf32x3B(c["B"].data_ptr(), K, Nl, True)
        ws_t = torch.empty(pkg.tf32x3_workspace_bytes(M, K), dtype=torch.uint8, device=dev)
        Ct = torch.empty((M, Nl), device=dev)
        tf_ms, _ = time_each(lambda: pkg.sgemm_joint_tf32x3(M, c["A"].data_ptr(), tb, Ct.data_ptr(), ws_t.data_ptr()),
                             reps)
        pkg.sgemm_joint(M, Nl, K, c["A"].data_ptr(), c["B"].data_ptr(), Cd.data_ptr(), c["bp"].data_ptr(), ws.data_ptr())
        tf_err = float(((Ct - Cd).abs().max() / Cd.abs().max().clamp_min(1e-30)).item())
        tf_live_k = tb.live_k
        tb.close()
        del ws_t, Ct
        density = bin(c["pat"]).count("1") / 8.0
        exec_flops = flops_dense_local * density           # uniform pattern: joint density = pattern density
        ref_cols = ref_kernel_times(M, Nl, K, c["A"], c["B"], both_ms, dev) if world == 1 else None
        pre_bytes = 4.0 * M * K + ap_bytes + 4.0 * M * K * density   # read A, write patterns, write live packed rows
        sweep[c["name"]] = {
            "joint_density": density,
            "ms_preprocess_a": pre_ms, "ms_preprocess_a_single_launch": pre_single_ms, "ms_gemm": gemm_ms, "ms_total": both_ms, "ms_cublas": cub_ms,
            "dense_equiv_tflops_incl_pre": flops_dense_local / (both_ms * 1e-3) / 1e12,
            "dense_equiv_tflops_gemm_only": flops_dense_local / (gemm_ms * 1e-3) / 1e12,
            "cublas_tflops": flops_dense_local / (cub_ms * 1e-3) / 1e12,
            "speedup_vs_cublas_incl_pre": cub_ms / both_ms,
            "executed_tflops": exec_flops / (gemm_ms * 1e-3) / 1e12,
            "frac_of_measured_ffma_peak": exec_flops / (gemm_ms * 1e-3) / 1e12 / ffma_peak,
            "frac_of_nominal_fp32_peak": exec_flops / (gemm_ms * 1e-3) / 1e12 / NOMINAL_FP32_TFLOPS,
            "preprocess_gbs": pre_bytes / (pre_ms * 1e-3) / 1e9,
            "preprocess_frac_of_hbm": pre_bytes / (pre_ms * 1e-3) / 1e9 / hbm_peak,
            "reference_kernels": ref_cols,
            "tf32x3": {"ms_total": tf_ms, "speedup_vs_cublas_incl_pre": cub_ms / tf_ms,
                       "speedup_vs_fp32_path": both_ms / tf_ms, "live_k": tf_live_k,
                       "rel_inf_vs_fp32_path": tf_err,
                       "dense_equiv_tflops_incl_pre": flops_dense_local / (tf_ms * 1e-3) / 1e12},
        }
        gemm_ms_sum += gemm_ms
        pre_ms_sum += pre_ms
        exec_flops_sum += exec_flops
    pkg.device_status()
    other = other_config_rows(pkg, torch, dev, time_each) if (world == 1 and workload == "c2" and not args.size
                                                            and not args.no_other_configs) else None
    achieved = exec_flops_sum / (gemm_ms_sum * 1e-3) / 1e12
    roofline = {
        "kernel": "esmm_joint_sgemm_packed_kernel", "bound": "fp32",
        "achieved": achieved, "peak": ffma_peak, "unit": "TFLOP/s", "frac": achieved / ffma_peak,
        "peak_source": "FFMA microbenchmark in this run (of measured); nominal 74.4 TFLOP/s at 1965 MHz",
        "flops_per_step": exec_flops_sum, "launches_per_step": len(cases),
        "traffic": TRAFFIC_BYTES_PER_LAUNCH.get((workload, M)),
        "traffic_note": "dram read+write bytes of the 100%-density launch from the ncu capture in profiles/",
        "share_of_step": gemm_ms_sum / (gemm_ms_sum + pre_ms_sum),
    }

    # the second kernel of the step, HBM bound: algorithmic bytes (read A, write the pattern bytes, write the live part of
    # the packed copy) over the launch-train time, against the measured copy bandwidth
    pre_bytes_sum = sum(4.0 * M * K + ap_bytes + 4.0 * M * K * v["joint_density"] for v in sweep.values())
    roofline_pre = {
        "kernel": "esmm_preprocess_a_pack64_kernel", "bound": "hbm", "achieved": pre_bytes_sum / (pre_ms_sum * 1e-3) / 1e9,
        "peak": hbm_peak, "unit": "GB/s", "frac": pre_bytes_sum / (pre_ms_sum * 1e-3) / 1e9 / hbm_peak,
        "peak_source": "MEASURED_PEAKS.json hbm_gbs (of %s)" % hbm_src, "bytes_per_step": pre_bytes_sum,
        "launches_per_step": len(cases), "traffic": None, "share_of_step": pre_ms_sum / (gemm_ms_sum + pre_ms_sum),
    }

    # ---- end to end through the host-buffer entry point (pinned host A and C, copies inside) ----
    e2e = None
    if dist is not None:
        # Multi-GPU: A lives in host memory once.  Every rank brings in 1 / world of its rows over its own PCIe
        # link, an all-gather over NVLink completes the replicas, then the rank's shard is computed and its
        # columns of C go back to host memory.
        c = cases[0]
        n_chunks = max(1, args.chunks)
        while n_chunks > 1 and M % (n_chunks * 128 * world):
            n_chunks -= 1
        rows_c = M // n_chunks                      # rows per chunk: whole tiles, equal slices per rank
        rows_s = rows_c // world
        dA = torch.empty((M, K), device=dev)
        hC = torch.empty((M, Nl), pin_memory=True)
        hA = []                                     # this rank's slice of every chunk, pinned
        for i in range(n_chunks):
            h = torch.empty((rows_s, K), pin_memory=True)
            h.copy_(c["A"][i * rows_c + rank * rows_s:i * rows_c + (rank + 1) * rows_s])
            hA.append(h)
        ws_c = [torch.empty(pkg.sgemm_joint_workspace_bytes(rows_c, K), dtype=torch.uint8, device=dev)
                for _ in range(n_chunks)]
        s_up, s_run, s_down = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
        ev_up = [torch.cuda.Event() for _ in range(n_chunks)]
        ev_run = [torch.cuda.Event() for _ in range(n_chunks)]

        def e2e_step():
            # chunks of rows: slice in + all-gather on one stream, packing + GEMM on a second, C out on a third
            for i in range(n_chunks):
                rows = slice(i * rows_c, (i + 1) * rows_c)
                with torch.cuda.stream(s_up):
                    sharding.upload_rows_replicated(hA[i], dA[rows], rank, world, dist)
                    ev_up[i].record(s_up)
                s_run.wait_event(ev_up[i])
                pkg.sgemm_joint(rows_c, Nl, K, dA[rows].data_ptr(), c["B"].data_ptr(), Cd[rows].data_ptr(),
                                c["bp"].data_ptr(), ws_c[i].data_ptr(), stream=s_run.cuda_stream)
                ev_run[i].record(s_run)
                s_down.wait_event(ev_run[i])
                with torch.cuda.stream(s_down):
                    hC[rows].copy_(Cd[rows], non_blocking=True)
            torch.cuda.synchronize()

        for _ in range(2):
            e2e_step()
        assert torch.equal(dA, c["A"])       # the replica assembled from the ranks' slices is A
        barrier()

        # where the end-to-end step's time goes: each phase of a step alone (all ranks at once, nothing overlapped),
        # device-timed on its own stream, max over ranks
        def phase_ms(fn, stream):
            barrier()
            a, b = ev(), ev()
            a.record(stream)
            fn()
            b.record(stream)
            barrier()
            return sharding.max_over_ranks(a.elapsed_time(b), dist, dev)

        def only_h2d():
            with torch.cuda.stream(s_up):
                for i in range(n_chunks):
                    r0 = i * rows_c + rank * rows_s
                    dA[r0:r0 + rows_s].copy_(hA[i], non_blocking=True)

        def only_allgather():
            with torch.cuda.stream(s_up):
                for i in range(n_chunks):
                    rows = dA[i * rows_c:(i + 1) * rows_c]
                    dist.all_gather_into_tensor(rows.view(-1), rows[rank * rows_s:(rank + 1) * rows_s].view(-1))

        def only_compute():
            for i in range(n_chunks):
                rows = slice(i * rows_c, (i + 1) * rows_c)
                pkg.sgemm_joint(rows_c, Nl, K, dA[rows].data_ptr(), c["B"].data_ptr(), Cd[rows].data_ptr(),
                                c["bp"].data_ptr(), ws_c[i].data_ptr(), stream=s_run.cuda_stream)

        def only_d2h():
            with torch.cuda.stream(s_down):
                hC.copy_(Cd, non_blocking=True)

        breakdown = {
            "h2d_ms": phase_ms(only_h2d, s_up), "allgather_ms": phase_ms(only_allgather, s_up),
            "compute_ms": phase_ms(only_compute, s_run), "d2h_ms": phase_ms(only_d2h, s_down),
            "h2d_bytes_per_rank": int(4 * M * K // world), "allgather_bytes_received_per_rank": int(4 * M * K * (world - 1) // world),
            "d2h_bytes_per_rank": int(4 * M * Nl),
            "note": "each phase alone, all ranks at once, max over ranks; the pipelined step overlaps them chunk by chunk",
        }
        breakdown["h2d_gbs_per_rank"] = breakdown["h2d_bytes_per_rank"] / (breakdown["h2d_ms"] * 1e-3) / 1e9
        breakdown["d2h_gbs_per_rank"] = breakdown["d2h_bytes_per_rank"] / (breakdown["d2h_ms"] * 1e-3) / 1e9
        breakdown["host_link_gbs_all_ranks"] = world * (breakdown["h2d_bytes_per_rank"] + breakdown["d2h_bytes_per_rank"]) / \
            ((breakdown["h2d_ms"] + breakdown["d2h_ms"]) * 1e-3) / 1e9
        e2e_steps = max(1, min(args.steps, 10))
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            e2e_step()
        barrier()
        dt = sharding.max_over_ranks(time.perf_counter() - t0, dist, dev)
        pkg.device_status()
        e2e = {"value": flops_dense * e2e_steps / dt / 1e12, "unit": "TFLOP/s",
               "h2d_bytes_per_step": int(4 * M * K), "d2h_bytes_per_step": int(4 * M * N),
               "ms_per_step": dt / e2e_steps * 1e3, "steps": e2e_steps, "chunks": n_chunks, "breakdown": breakdown,
               "note": "whole job per step, in row chunks on three streams: every rank copies 1 / world of the chunk's "
                       "rows of A from pinned host memory, all-gather over NVLink, packing + GEMM on the rank's column "
                       "shard, the chunk of C back to pinned host memory; B and its patterns resident"}
        del dA, hA, hC, ws_c
    elif rank == 0:
        import ctypes as C
        plans = []
        for c in cases:
            hB = c["B"].cpu()
            plan = C.c_void_p()
            pkg.check(L.esmm_plan_create(M, Nl, K, hB.data_ptr(), args.chunks, C.byref(plan)), "esmm_plan_create")
            hA = torch.empty((M, K), pin_memory=True)
            hA.copy_(c["A"])
            plans.append((plan, hA, torch.empty((M, Nl), pin_memory=True)))
            del hB

        def e2e_step():
            # the step's GEMMs are submitted together (the copies of one overlap the kernels of another)
            # and the step ends when every result is in host memory
            for plan, hA, hC in plans:
                pkg.check(L.esmm_plan_submit(plan, hA.data_ptr(), hC.data_ptr()), "esmm_plan_submit")
            for plan, _, _ in plans:
                pkg.check(L.esmm_plan_wait(plan), "esmm_plan_wait")

        for _ in range(2):
            e2e_step()
        barrier()
        e2e_steps = max(1, min(args.steps, 10))
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            e2e_step()
        barrier()
        dt = time.perf_counter() - t0
        if dist is not None:
            dt = sharding.max_over_ranks(dt, dist, dev)
        for plan, _, _ in plans:
            L.esmm_plan_destroy(plan)
        e2e = {"value": len(cases) * flops_dense * e2e_steps / dt / 1e12, "unit": "TFLOP/s",
               "h2d_bytes_per_step": int(len(cases) * 4 * M * K), "d2h_bytes_per_step": int(len(cases) * 4 * M * Nl),
               "ms_per_step": dt / e2e_steps * 1e3, "steps": e2e_steps, "chunks": args.chunks,
               "note": "esmm_plan_submit x cases + esmm_plan_wait per step: pinned host A in, pinned host C out, "
                       "B and its patterns resident"}

    # ---- optional gather of C to every rank, timed separately ----
    gather = None
    if dist is not None:
        def interleave(staging, out, m, n, w):
            pkg.check(L.esmm_interleave_shards(staging.data_ptr(), out.data_ptr(), m, n, w, 0), "interleave")
        sharding.gather_columns(Cd, shard, dist, interleave)
        barrier()
        a, b = ev(), ev()
        a.record()
        full = sharding.gather_columns(Cd, shard, dist, interleave)
        b.record()
        barrier()
        gather = {"ms": sharding.max_over_ranks(a.elapsed_time(b), dist, dev), "bytes": int(4 * M * N)}
        del full

    # ---- CPU baseline (rank 0, N = 1 only): bounded row sample ----
    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu:
        cpu = CpuSgemm(M, N, K, 0xFF)
        rows = cpu.calibrate(target_s=12.0)
        dt = cpu.run(rows)
        sample = f"{rows} of {M} rows of C (all {N} columns, full K), once; extrapolates linearly in rows"
        cpu_baseline = {"value": 2.0 * rows * N * K / dt / 1e12, "unit": "TFLOP/s", "cores": cpu.threads,
                        "kind": cpu.kind, "sample": sample, "seconds": dt}

    # ---- the multi-GPU workload on this one GPU: the base the --gpus N > 1 lines (workload c5) compare with ----
    scaling_base = None
    if rank == 0 and not args.no_scaling_base and (workload == "c2" or world > 1) and not args.size:
        S5 = 16384
        A5 = torch.empty((S5, S5), device=dev)
        B5 = torch.empty((S5, S5), device=dev)
        C5 = torch.empty((S5, S5), device=dev)
        pkg.fill_normal(A5.data_ptr(), S5, S5, 0, 1, mode=1, pattern=0x03)
        pkg.fill_normal(B5.data_ptr(), S5, S5, 1, 1000, mode=1, pattern=0x03)
        bp5 = torch.empty(L.esmm_b_pattern_bytes(S5, S5), dtype=torch.uint8, device=dev)
        pkg.preprocess_b(B5.data_ptr(), S5, S5, bp5.data_ptr())
        ws5 = torch.empty(pkg.sgemm_joint_workspace_bytes(S5, S5), dtype=torch.uint8, device=dev)

        def step5():
            pkg.sgemm_joint(S5, S5, S5, A5.data_ptr(), B5.data_ptr(), C5.data_ptr(), bp5.data_ptr(), ws5.data_ptr())

        for _ in range(3):
            step5()
        torch.cuda.synchronize()
        n5 = 5
        a5, b5 = ev(), ev()
        a5.record()
        for _ in range(n5):
            step5()
        b5.record()
        torch.cuda.synchronize()
        pkg.device_status()
        ms5 = a5.elapsed_time(b5) / n5
        scaling_base = {"workload": "c5: M=N=K=16384 FP32, pattern 11000000, on this one GPU", "ms_per_step": ms5,
                        "value": 2.0 * S5 ** 3 / (ms5 * 1e-3) / 1e12, "unit": "TFLOP/s", "steps": n5,
                        "note": "bench.py --gpus N > 1 runs this workload column-sharded; its value / this value is the "
                                "speed-up over one GPU (the N = 1 headline is workload c2, a different problem)"}
        del A5, B5, C5, bp5, ws5
    if dist is not None:
        barrier()   # the other ranks wait for rank 0's single-GPU run

    if rank == 0:
        line = {
            "metric": METRIC_C2 if workload == "c2" else METRIC_C5,
            "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong" if world > 1 else "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {
                "workload": ("c2: M=N=K=%d FP32, N(0,1), uniform patterns 11111111/11110000/11000000/10000000 on A's "
                             "K columns and B's K rows; step = the 4 densities once" % M) if workload == "c2" else
                            ("c5: M=N=K=%d FP32, N(0,1), uniform pattern 11000000; B, its cached patterns and C "
                             "column-sharded over %d GPUs, A and its preprocessing replicated" % (M, world)),
                "M": M, "N": N, "K": K, "patterns": [p for p, _ in pats], "b_patterns": "cached (offline)",
                "a_patterns": "per call (packing preprocess inside the timed region)",
                "l2": "inputs larger than L2: %.0f MB of A/B/C/packed-A touched per step vs 126 MB L2"
                      % (len(cases) * (2 * 4.0 * M * K + 4.0 * K * Nl) / 1e6 + 4.0 * M * Nl / 1e6),
                "parallelism": "N-column shards, no collective" if world > 1 else "1 GPU",
            },
            "sweep": sweep, "other_configs": other, "roofline": roofline, "roofline_preprocess": roofline_pre,
            "cpu_baseline": cpu_baseline, "e2e": e2e,
            "gpu_launches": int(args.steps * len(cases) * 2), "clocks": clocks,
            "ffma_peak_tflops_measured": ffma_peak, "hbm_peak_gbs": hbm_peak, "hbm_peak_source": hbm_src,
            "sm_count": sms, "gather_c": gather, "scaling_base": scaling_base,
        }
        cfg = line["config"]
        # compact copies inside `config`: ours / cuBLAS / reference id 29 per density, the one-GPU base of the
        # sharded workload, the shard check
        cfg["ms_ours_cublas_ref29"] = {
            k: [round(v["ms_total"], 4), round(v["ms_cublas"], 4),
                round(v["reference_kernels"]["ms_ref_id29"], 4) if v.get("reference_kernels") and
                "ms_ref_id29" in v["reference_kernels"] else None] for k, v in sweep.items()}
        if other:
            cfg["ms_ours_cublas_ref29_other"] = {
                k: [round(v["ms_total"], 4), round(v["ms_cublas"], 4),
                    round(v["reference_kernels"]["ms_ref_id29"], 4) if v.get("reference_kernels") and
                    "ms_ref_id29" in v["reference_kernels"] else None] for k, v in other.items()}
        if scaling_base:
            cfg["scaling_base_tflops"] = scaling_base["value"]
            cfg["scaling_base_ms_per_step"] = scaling_base["ms_per_step"]
            cfg["scaling_base_workload"] = scaling_base["workload"]
            if workload == "c5":
                cfg["speedup_vs_1gpu"] = value / scaling_base["value"]
        if shard_check is not None:
            cfg["shard_check"] = shard_check
        # the optional 3xTF32 tensor-core entry point on the same inputs, as one step of the same cases: not `value`
        # (its results are inside the 1e-4 tolerance but not the FP32 path's bits), rank 0's shard at N > 1
        tf_ms = sum(v["tf32x3"]["ms_total"] for v in sweep.values())
        line["tensor_core_variant"] = {
            "entry": "esmm_sgemm_joint_tf32x3", "ms_per_step_this_rank": tf_ms,
            "dense_equiv_tflops_this_rank": len(cases) * flops_dense_local / (tf_ms * 1e-3) / 1e12,
            "speedup_vs_fp32_path": sum(v["ms_total"] for v in sweep.values()) / tf_ms,
            "max_rel_inf_vs_fp32_path": max(v["tf32x3"]["rel_inf_vs_fp32_path"] for v in sweep.values()),
        }
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the dominant kernel (the
# 100%-density launch of the sweep), from the ncu capture summarised in
# profiles/packed_gemm_4096_density100.txt; None for workloads without a capture.
TRAFFIC_BYTES_PER_LAUNCH = {("c2", 4096): 336519680 + 54495744}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=None, choices=["c2", "c5"])
    ap.add_argument("--size", type=int, default=None, help="override M = N = K (experiments only)")
    ap.add_argument("--chunks", type=int, default=8, help="row chunks of the host-buffer pipeline")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-scaling-base", action="store_true", help="skip the single-GPU run of the multi-GPU workload")
    ap.add_argument("--no-check", action="store_true", help="skip the untimed oracle check of the shards (N > 1)")
    ap.add_argument("--no-other-configs", action="store_true", help="skip the config 3 / config 4 comparison rows")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
