"""Generates the golden fixtures of tests/golden/ from the UNMODIFIED reference
(oracle/_ref/libesmm_ref.so, built by oracle/Makefile from the reference tree).

  python tests/golden/make_golden.py cpu   # needs no GPU: reference host functions
  python tests/golden/make_golden.py gpu [output directory]   # needs a GPU: reference pattern kernels + kernel id 29

cpu -> ref_cpu.npz : inputs drawn by the reference's own rand()-based generators
                     (randomize_matrix_A_blocklevel<8,32>, randomize_matrix_B_blocklevel_fixed<8,32>,
                     randomize_matrix_with_pattern, randomize_matrix_unstructured, randomize_matrix_A<8,8>),
                     the reference CPU SGEMM (matrixMultiplyCPU) of them, the reference's kernel-selection
                     parser / kernel names, and its literal PatternLUT table.
gpu -> ref_gpu.npz : for seeded inputs (recreated by seed in the tests, not stored), the pattern
                     bytes of preprocess_ab<8,32,32> and the C of esmm_ab_optimized_v3 as run on a B200.
The gpu mode writes ref_gpu.npz into the output directory given (default: tests/golden/ itself), for the case
that the GPU machine is not the one that holds the repository.
"""
from __future__ import annotations

import ctypes
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))
import oracle  # noqa: E402
import workloads  # noqa: E402

# (name, M, N, K, generator, args): recreated identically by tests/test_golden.py
GPU_CASES = [
    ("uniform_0f_256", 256, 256, 256, "uniform_pattern", dict(pattern=0x0F, seed=0)),
    ("uniform_01_128x256x512", 128, 256, 512, "uniform_pattern", dict(pattern=0x01, seed=2)),
    ("tile_random_256x384x512", 256, 384, 512, "tile_random", dict(pA=0.5, pB=0.5, seed=3, gran_a=32, gran_b=32)),
    ("tile_random_sparse_512", 512, 512, 1024, "tile_random", dict(pA=0.2, pB=0.3, seed=4, gran_a=64, gran_b=64)),
    ("llm_mlp_128x512x1024", 128, 512, 1024, "llm_mlp", dict(seed=5)),
    ("all_bytes_64x128", 64, 128, 2048, "all_byte_values", dict(seed=6)),
]


def make_case(gen: str, M: int, N: int, K: int, args: dict):
    if gen == "all_byte_values":
        return workloads.all_byte_values(M, N, **args)
    return getattr(workloads, gen)(M, N, K, **args)


def parse_pattern_lut(path: str):
    """The 256 `{count, {o0, ..., o7}}` initialisers of PATTERN_LUT_BK8 (include/pattern_lut.cuh), in order."""
    import re
    text = open(path).read()
    body = text[text.index("PATTERN_LUT_BK8"):]
    rows = re.findall(r"\{\s*(\d+)\s*,\s*\{([^}]*)\}\s*\}", body)
    assert len(rows) == 256, len(rows)
    cnt = np.array([int(c) for c, _ in rows], np.uint8)
    off = np.array([[int(x) for x in o.split(",")] for _, o in rows], np.uint8)
    assert off.shape == (256, 8)
    return cnt, off


def cpu() -> None:
    R = oracle.ref()
    out = {}
    M, N, K = 64, 128, 64
    A = np.zeros((M, K), np.float32)
    B = np.zeros((K, N), np.float32)
    # driver.cu:385,389: --blockwise, seeds 12345 / 12346, 50 % block sparsity
    R.ref_randomize_A_blocklevel_8_32(A, M, K, 50.0, 12345)
    R.ref_randomize_B_blocklevel_8_32(B, K, N, 50.0, 12346)
    C = np.zeros((M, N), np.float32)
    R.ref_matrixMultiplyCPU(A, B, C, M, N, K)
    out.update(blk_A=A, blk_B=B, blk_C=C)
    # driver.cu:403-406: default pattern mode (column index mod 8), rand() state continues
    A2 = np.zeros((32, 64), np.float32)
    B2 = np.zeros((64, 32), np.float32)
    R.ref_srand(1)
    R.ref_randomize_with_pattern(A2, 32, 64, b"11110000")
    R.ref_randomize_with_pattern(B2, 64, 32, b"11110000")
    C2 = np.zeros((32, 32), np.float32)
    R.ref_matrixMultiplyCPU(A2, B2, C2, 32, 32, 64)
    out.update(pat_A=A2, pat_B=B2, pat_C=C2)
    # driver.cu:401-402: --random (37.5 % unstructured, seeds 12345 / 12346)
    A3 = np.zeros((48, 40), np.float32)
    B3 = np.zeros((40, 56), np.float32)
    R.ref_randomize_unstructured(A3, 48, 40, 37.5, 12345)
    R.ref_randomize_unstructured(B3, 40, 56, 37.5, 12346)
    out.update(rnd_A=A3, rnd_B=B3)
    # driver.cu:382: --blockwise with kernel 21 selected: 8-row tiles of A
    A4 = np.zeros((64, 64), np.float32)
    R.ref_randomize_A_8_8(A4, 64, 64, 75.0, 12345)
    out.update(a8_A=A4)
    # include/pattern_lut.cuh: the literal table, read as text (it is __constant__ device data)
    cnt, off = parse_pattern_lut(os.path.join(oracle.ref_root(), "include", "pattern_lut.cuh"))
    out.update(lut_count=cnt, lut_offsets=off)
    # parser + names
    sels = ["29", "29,15", "14-17", "all", "20,21,25", "1-100", "99", "15,99,29"]
    buf = (ctypes.c_int * 32)()
    parsed = []
    for s in sels:
        n = R.ref_parse_kernel_selection(s.encode(), buf, 32)
        parsed.append(",".join(str(buf[i]) for i in range(max(n, 0))))
    out["selections"] = np.array(sels)
    out["parsed"] = np.array(parsed)
    ids = [14, 15, 16, 17, 20, 21, 25, 26, 27, 28, 29, 30, 31]
    out["name_ids"] = np.array(ids)
    out["names"] = np.array([R.ref_get_kernel_name(i).decode() for i in ids])
    np.savez_compressed(os.path.join(HERE, "ref_cpu.npz"), **out)
    print("wrote", os.path.join(HERE, "ref_cpu.npz"))


def gpu() -> None:
    import torch
    R = oracle.ref()
    out = {}
    for name, M, N, K, gen, args in GPU_CASES:
        A, B = make_case(gen, M, N, K, args)
        M, K = A.shape
        N = B.shape[1]
        dA, dB = torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda()
        ra = torch.zeros((M // 32, K // 8), dtype=torch.uint8, device="cuda")
        rb = torch.zeros((N // 32, K // 8), dtype=torch.uint8, device="cuda")
        e = R.ref_preprocess_ab_32(dA.data_ptr(), dB.data_ptr(), M, N, K, ra.data_ptr(), rb.data_ptr())
        assert e == 0, e
        out[name + ".a_pat"] = ra.cpu().numpy()
        out[name + ".b_pat"] = rb.cpu().numpy()
        if M % 64 == 0 and N % 128 == 0:  # the reference kernel's own shape limits
            dC = torch.zeros((M, N), device="cuda")
            e = R.ref_esmm_v3_launch(M, N, K, dA.data_ptr(), dB.data_ptr(), dC.data_ptr(), ra.data_ptr(),
                                     rb.data_ptr())
            torch.cuda.synchronize()
            assert e == 0, e
            out[name + ".C"] = dC.cpu().numpy()
        out[name + ".shape"] = np.array([M, N, K])
    dst = sys.argv[2] if len(sys.argv) > 2 else HERE
    np.savez_compressed(os.path.join(dst, "ref_gpu.npz"), **out)
    print("wrote", os.path.join(dst, "ref_gpu.npz"))


if __name__ == "__main__":
    {"cpu": cpu, "gpu": gpu}[sys.argv[1]]()
