"""Sweep script (esmm-research_b200/sweep.py) and the cuSPARSE comparison (esmm_cusparse_spmm, cusparse_bench)."""
import csv
import ctypes as C
import importlib.util
import os
import subprocess

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "esmm-research_b200")


@pytest.fixture(scope="module")
def sweep(pkg):
    spec = importlib.util.spec_from_file_location("esmm_sweep", os.path.join(PKG, "sweep.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_sweep_planning_and_parsing(sweep, tmp_path, capsys):
    assert sweep.valid_pattern("11110000") and not sweep.valid_pattern("1111") and not sweep.valid_pattern("1111000x")
    assert sweep.density("11000000") == 0.25
    pts = sweep.plan_points([1024, 2048], ["11111111", "10000000"])
    assert pts == [(1024, "11111111", "11111111"), (1024, "10000000", "10000000"),
                   (2048, "11111111", "11111111"), (2048, "10000000", "10000000")]
    assert sweep.plan_points([512], ["11111111", "11110000"], pattern_a="11000000") == \
        [(512, "11000000", "11111111"), (512, "11000000", "11110000")]
    assert sweep.plan_points([512], ["11111111"], "11000000", "10000000") == [(512, "11000000", "10000000")]
    cmd = sweep.driver_command("29,15", 5, 1024, "11110000", "11000000", "uniform")
    assert cmd[1:] == ["29,15", "5", "--size", "1024", "--pattern-a", "11110000", "--pattern-b", "11000000", "--no-check",
                       "--json", "--uniform"]
    text = ('Kernel time: 1.0 ms (avg: 0.5 ms)\n'
            '{"kernel": 29, "M": 1024, "N": 1024, "K": 1024, "runs": 5, "avg_ms": 0.041000, "dense_equiv_tflops": 52.378, '
            '"status": 0, "passed": true, "cpu_rel_inf": -1}\nSummary: 1/1 kernels completed (no verification)\n')
    rows = sweep.parse_driver_output(text, 1024, "11110000", "11110000", "uniform")
    assert rows == [{"kernel": 29, "size": 1024, "pattern_a": "11110000", "pattern_b": "11110000", "mode": "uniform",
                     "density_a": 0.5, "density_b": 0.5, "runs": 5, "avg_ms": "0.0410", "dense_equiv_tflops": "52.38",
                     "status": 0}]
    assert sweep.parse_sparse_row("4096,0.5000,100.000,200.000,10.00,5.00\n")["total_us"] == "200.000"
    assert sweep.parse_sparse_row("size,density,spmm_us\n") is None
    assert sweep.main(["-k", "29", "--sparsity", "1111"]) == 1 and "must be 8 characters" in capsys.readouterr().out
    assert sweep.main(["-k", "29", "-b", "-u"]) == 1


@pytest.mark.gpu
def test_sweep_runs_the_driver(sweep, cuda, tmp_path):
    out = tmp_path / "s.csv"
    assert sweep.main(["-k", "29,15", "--sizes", "256,512", "--sparsity", "11110000,10000000", "--uniform", "--runs", "2",
                       "--cusparse", "-o", str(out)]) == 0
    with open(out) as f:
        rows = list(csv.DictReader(f))
    assert len(rows) == 8 and {r["kernel"] for r in rows} == {"29", "15"} and all(float(r["avg_ms"]) > 0 for r in rows)
    with open(tmp_path / "s_cusparse.csv") as f:
        srows = list(csv.DictReader(f))
    assert len(srows) == 4 and all(float(r["rel_diff"]) <= 1e-4 for r in srows)


@pytest.mark.gpu
def test_cusparse_spmm_matches_joint_kernel(cuda, pkg, oracle_mod):
    import workloads
    M, N, K = 256, 384, 512
    A, B = workloads.tile_random(M, N, K, 0.3, 1.0, seed=9, gran_a=64, gran_b=32)
    dA, dB = cuda.from_numpy(A).cuda(), cuda.from_numpy(B).cuda()
    dC = cuda.zeros((M, N), device="cuda")
    spmm, total, nnz = C.c_float(0), C.c_float(0), C.c_longlong(0)
    L = pkg.lib()
    pkg.check(L.esmm_cusparse_spmm(M, N, K, dA.data_ptr(), dB.data_ptr(), dC.data_ptr(), 3, C.byref(spmm), C.byref(total),
                                   C.byref(nnz)), "esmm_cusparse_spmm")
    assert nnz.value == int(np.count_nonzero(A)) and 0 < spmm.value <= total.value * 1.5
    assert oracle_mod.rel_inf_err(dC.cpu().numpy(), oracle_mod.gemm_joint(A, B)) <= 1e-4
    assert L.esmm_cusparse_spmm(M, N, K, None, dB.data_ptr(), dC.data_ptr(), 1, None, None, None) == pkg.ERR_NULL
    assert L.esmm_cusparse_spmm(M, N, K, dA.data_ptr(), dB.data_ptr(), dC.data_ptr(), 0, None, None, None) == pkg.ERR_SHAPE
    # the standalone binary: header and one row in the reference's format
    exe = os.path.join(PKG, "cusparse_bench")
    assert subprocess.run([exe, "--header"], capture_output=True, text=True).stdout.strip() == \
        "size,density,spmm_us,total_us,spmm_gflops,total_gflops"
    row = subprocess.run([exe, "--size", "512", "--density", "0.25", "--runs", "2"], capture_output=True, text=True).stdout
    parts = row.strip().split(",")
    assert len(parts) == 6 and parts[0] == "512" and float(parts[4]) > 0
