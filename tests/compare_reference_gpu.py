"""Side-by-side timing of this library and of the UNMODIFIED reference kernels on the same device
buffers (needs a GPU and oracle/_ref/libesmm_ref.so, which oracle/Makefile builds from the reference
tree).  Not collected by pytest; run it by hand:

    python tests/compare_reference_gpu.py [size]

Per uniform pattern of config 2 it prints: the reference's pattern preprocessor + kernel id 29
(recompiled for sm_100a, its own launch configuration), cuBLAS SGEMM, and this library's per-call
path (packing preprocess of A + packed GEMM, B patterns cached), each as the median of 10 CUDA-event
timings after 3 warm-ups, and whether the three C matrices are bit-identical.
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import __graft_entry__ as g  # noqa: E402
import oracle  # noqa: E402


def timeit(fn, iters=10, warm=3):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    return float(np.median(ts))


def main():
    S = int(sys.argv[1]) if len(sys.argv) > 1 else 4096
    pkg = g.load_package()
    L, R = pkg.lib(), oracle.ref()
    torch.cuda.set_device(0)
    dA = torch.empty((S, S), device="cuda")
    dB = torch.empty((S, S), device="cuda")
    c_ours, c_ref, c_blas = (torch.empty((S, S), device="cuda") for _ in range(3))
    bp = torch.empty(L.esmm_b_pattern_bytes(S, S), dtype=torch.uint8, device="cuda")
    ws = torch.empty(pkg.sgemm_joint_workspace_bytes(S, S), dtype=torch.uint8, device="cuda")
    ra = torch.empty((S // 32, S // 8), dtype=torch.uint8, device="cuda")
    rb = torch.empty_like(ra)
    print(f"M = N = K = {S}, FP32, N(0,1), uniform patterns; times in ms")
    print(f"{'pattern':10s} {'ref pre A+B':>12s} {'ref id 29':>10s} {'cuBLAS':>8s} {'ours pre A':>11s} {'ours GEMM':>10s} "
          f"{'ours total':>11s} {'vs ref 29':>10s} {'vs cuBLAS':>10s}  bit-identical(ref29, cuBLAS)")
    for name, pat in (("11111111", 0xFF), ("11110000", 0x0F), ("11000000", 0x03), ("10000000", 0x01)):
        pkg.fill_normal(dA.data_ptr(), S, S, 0, 1, mode=1, pattern=pat)
        pkg.fill_normal(dB.data_ptr(), S, S, 1, 2, mode=1, pattern=pat)
        pkg.preprocess_b(dB.data_ptr(), S, S, bp.data_ptr())
        t_refpre = timeit(lambda: R.ref_preprocess_ab_32(dA.data_ptr(), dB.data_ptr(), S, S, S, ra.data_ptr(), rb.data_ptr()))
        t_ref = timeit(lambda: R.ref_esmm_v3_launch(S, S, S, dA.data_ptr(), dB.data_ptr(), c_ref.data_ptr(), ra.data_ptr(),
                                                    rb.data_ptr()))
        t_blas = timeit(lambda: pkg.cublas_sgemm(S, S, S, dA.data_ptr(), dB.data_ptr(), c_blas.data_ptr()))
        n_ap = ra.numel()
        pack = ws[(n_ap + 255) & ~255:]
        t_pre = timeit(lambda: pkg.preprocess_a_packed(dA.data_ptr(), S, S, ws.data_ptr(), pack.data_ptr()))
        t_gemm = timeit(lambda: pkg.gemm_ab_packed(S, S, S, pack.data_ptr(), dB.data_ptr(), c_ours.data_ptr(), ws.data_ptr(),
                                                   bp.data_ptr()))
        t_tot = timeit(lambda: pkg.sgemm_joint(S, S, S, dA.data_ptr(), dB.data_ptr(), c_ours.data_ptr(), bp.data_ptr(),
                                               ws.data_ptr()))
        pkg.device_status()
        same = (bool(torch.equal(c_ours, c_ref)), bool(torch.equal(c_ours, c_blas)))
        pats_same = bool(torch.equal(ws[:n_ap].view(ra.shape), ra)) and bool(torch.equal(bp.view(rb.shape), rb))
        print(f"{name:10s} {t_refpre:12.4f} {t_ref:10.4f} {t_blas:8.4f} {t_pre:11.4f} {t_gemm:10.4f} {t_tot:11.4f} "
              f"{(t_ref) / t_tot:9.2f}x {t_blas / t_tot:9.2f}x  {same}  patterns equal: {pats_same}")


if __name__ == "__main__":
    main()
