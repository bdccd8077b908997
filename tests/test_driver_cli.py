"""The exec_b200 command line: same grammar, messages and exit codes as the reference driver
(driver.cu:142-487), plus the additive generator flags."""
import json
import os
import subprocess

import numpy as np
import pytest


def run(pkg, *args):
    if not os.path.exists(pkg.EXE_PATH):
        import __graft_entry__ as g
        g.build()
    p = subprocess.run([pkg.EXE_PATH, *args], capture_output=True, text=True, timeout=600)
    return p.returncode, p.stdout + p.stderr


# ---- argument handling: no GPU needed ---------------------------------------------------------
def test_help_and_argument_errors(pkg):
    rc, out = run(pkg, "--help")
    assert rc == 0 and "Usage:" in out and "--blockwise" in out and "29:" in out
    rc, out = run(pkg, "99", "1")
    assert rc == 1 and "Error: Invalid kernel selection '99'" in out
    rc, out = run(pkg, "29", "1", "--pattern", "1100")
    assert rc == 1 and "Pattern must be exactly 8 characters" in out
    rc, out = run(pkg, "29", "1", "--pattern", "1100000x")
    assert rc == 1 and "Pattern must contain only '0' and '1' characters" in out
    rc, out = run(pkg, "29", "0")
    assert rc == 1 and "Number of runs must be positive" in out
    rc, out = run(pkg, "29", "1", "--size", "-4")
    assert rc == 1 and "Size must be positive" in out
    rc, out = run(pkg, "29", "1", "--size")
    assert rc == 1 and "--size requires an argument" in out
    rc, out = run(pkg, "29", "1", "--load-b", "w.bin")
    assert rc == 1 and "--dims M K N required with --load-a / --load-b" in out
    # the multi-GPU flags are checked on the host before any device is touched
    rc, out = run(pkg, "29", "1", "--gpus", "3", "--size", "4096")
    assert rc == 1 and "does not split into 3 column shards" in out
    rc, out = run(pkg, "29,15", "1", "--gpus", "2", "--size", "4096")
    assert rc == 1 and "--gpus runs kernel 29 only" in out
    rc, out = run(pkg, "29", "1", "--gather", "--size", "256")
    assert rc == 1 and "--gather needs --gpus" in out
    rc, out = run(pkg, "29", "1", "--gpus", "0")
    assert rc == 1 and "--gpus must be positive" in out
    rc, out = run(pkg, "29", "1", "--tune", "NO_SUCH_HOOK=1")
    assert rc == 1 and "--tune wants NAME=VALUE with a name the library knows" in out
    rc, out = run(pkg, "29", "1", "--tune", "PRODUCER_WARPS")
    assert rc == 1 and "--tune wants NAME=VALUE" in out


# ---- runs ---------------------------------------------------------------------------------------
@pytest.mark.gpu
def test_blockwise_run_with_cublas_check(pkg, cuda):
    rc, out = run(pkg, "29,15", "2", "--blockwise", "--pattern", "11110000", "--size", "512", "--skip-stats")
    assert rc == 0, out
    assert out.count("PASSED") == 2 and "Summary: 2/2 kernels passed" in out
    assert out.count("Kernel time:") == 2 and "=== Skip Stats: K29 ===" in out
    assert "Kernel 29 (ESMM A+B Optimized V3 (K26 + templated smem + float2 A-loads)): PASSED" in out


@pytest.mark.gpu
@pytest.mark.parametrize("shape", ["3", "0", "7"])
def test_tune_flag_pins_the_launch_shape(pkg, cuda, shape):
    """`--tune PRODUCER_WARPS=v` (additive): scattered 32-granular patterns through each launch shape of the tiled kernel."""
    rc, out = run(pkg, "29", "3", "--tile-random", "0.2", "0.2", "--tile-gran", "32", "--size", "512", "--cpu-check",
                  "--tune", "PRODUCER_WARPS=" + shape)
    assert rc == 0, out
    assert "PASSED" in out and "CPU SGEMM check" in out


@pytest.mark.gpu
def test_uniform_cpu_check_json(pkg, cuda):
    rc, out = run(pkg, "29", "2", "--uniform", "--pattern", "10000000", "--size", "512", "--cpu-check", "--json")
    assert rc == 0, out
    line = json.loads([l for l in out.splitlines() if l.startswith("{")][0])
    assert line["kernel"] == 29 and line["passed"] is True and 0 <= line["cpu_rel_inf"] <= 1e-4
    assert "CPU SGEMM check" in out


@pytest.mark.gpu
def test_default_pattern_random_and_verbose_modes(pkg, cuda):
    rc, out = run(pkg, "29", "1", "--size", "256", "--pattern", "11110000", "--verbose")
    assert rc == 0 and "Sparsity mode: PATTERN-BASED (column-wise)" in out and "Status: PASSED" in out
    rc, out = run(pkg, "25-29", "1", "--size", "256", "--random", "--no-check")
    assert rc == 0 and out.count("COMPLETED (no verification)") == 5
    assert "Summary: 5/5 kernels completed (no verification)" in out
    rc, out = run(pkg, "29", "1", "--size", "256", "--tile-random", "0.3", "0.7", "--seed", "7")
    assert rc == 0 and "PASSED" in out


@pytest.mark.gpu
def test_load_raw_weights(pkg, cuda, tmp_path):
    M, K, N = 128, 256, 384
    rng = np.random.default_rng(0)
    B = rng.standard_normal((K, N), dtype=np.float32)
    B[(np.arange(K) % 8) >= 2] = 0.0
    path = tmp_path / "w.bin"
    B.tofile(path)
    rc, out = run(pkg, "29,15", "1", "--load-b", str(path), "--dims", str(M), str(K), str(N))
    assert rc == 0 and "Summary: 2/2 kernels passed" in out
    (tmp_path / "short.bin").write_bytes(b"\0" * 100)
    rc, out = run(pkg, "29", "1", "--load-b", str(tmp_path / "short.bin"), "--dims", str(M), str(K), str(N))
    assert rc == 1 and "Error: expected" in out
    rc, out = run(pkg, "29", "1", "--load-b", str(tmp_path / "none.bin"), "--dims", str(M), str(K), str(N))
    assert rc == 1 and "Error: cannot open" in out


@pytest.mark.gpu
def test_single_operand_ids(pkg, cuda):
    """Ids 14, 16, 17 run through the joint kernel: default column-pattern data (A's K columns masked by
    the pattern, which is what id 14 assumes), verified against cuBLAS like the reference driver does."""
    rc, out = run(pkg, "14-17", "2", "--size", "256", "--pattern", "11110000")
    assert rc == 0 and "Summary: 4/4 kernels passed" in out, out
    # id 14 has kernels for 1, 2, 4, 6, 8 live k only: with 3 nothing is launched and C stays zero
    rc, out = run(pkg, "14", "1", "--size", "256", "--pattern", "11100000")
    assert rc == 1 and "Verification failed" in out and "Summary: 0/1 kernels passed" in out


@pytest.mark.gpu
def test_b_pattern_cache_file(pkg, cuda, tmp_path):
    """--cache-b: first run computes and saves <weights>.bpat, the second loads it; a file written for
    another shape is recomputed.  The saved bytes equal the oracle's B patterns."""
    import oracle
    M, K, N = 128, 256, 384
    rng = np.random.default_rng(1)
    B = rng.standard_normal((K, N), dtype=np.float32)
    B[(np.arange(K) % 8) >= 3] = 0.0
    path = tmp_path / "w.bin"
    B.tofile(path)
    args = ("29", "2", "--load-b", str(path), "--dims", str(M), str(K), str(N), "--cache-b")
    rc, out = run(pkg, *args)
    assert rc == 0 and "B patterns: computed and saved to" in out and "PASSED" in out
    raw = (tmp_path / "w.bin.bpat").read_bytes()
    assert raw[:8] == b"ESMMBPT1"
    assert np.array_equal(np.frombuffer(raw[32:], np.uint8).reshape(N // 32, K // 8), oracle.preprocess_b(B))
    rc, out = run(pkg, *args)
    assert rc == 0 and "B patterns: loaded from" in out and "PASSED" in out
    rc, out = run(pkg, "29", "1", "--load-b", str(path), "--dims", str(M), str(K // 2), str(2 * N), "--cache-b")
    assert "written for another shape, recomputing" in out


@pytest.mark.gpu
def test_gpus_flag_on_one_gpu(pkg, cuda):
    """--gpus 1: the sharded launcher's degenerate case (one shard) through the CLI, verified against cuBLAS and
    the CPU SGEMM like any other run."""
    rc, out = run(pkg, "29", "2", "--gpus", "1", "--uniform", "--pattern", "11000000", "--size", "512", "--cpu-check", "--json")
    assert rc == 0, out
    assert "1 GPUs, column shards of 512" in out and "Kernel 29" in out and "PASSED" in out
    line = json.loads([l for l in out.splitlines() if l.startswith("{")][0])
    assert line["gpus"] == 1 and line["passed"] is True and len(line["ms_per_gpu"]) == 1 and 0 <= line["cpu_rel_inf"] <= 1e-4


@pytest.mark.gpu
def test_reference_driver_runs_against_this_library(pkg, cuda, oracle_mod):
    """The reference's OWN driver.cu, byte for byte, built against this repository's include/ and libesmm_b200
    (oracle/_ref/exec_swapped, made by oracle/Makefile where the reference tree is at hand): its main(), its generators
    by name, its cuBLAS reference, its switch over the kernel ids and its PASSED / FAILED lines - with this library
    underneath.  The header swap at run time, not only at compile time."""
    exe = oracle_mod.SWAPPED_EXE
    if not os.path.exists(exe):
        pytest.skip("oracle/_ref/exec_swapped not built (needs the reference tree at build time)")

    def run_ref(*args):
        p = subprocess.run([exe, *args], capture_output=True, text=True, timeout=600)
        return p.returncode, p.stdout + p.stderr
    rc, out = run_ref("29,15", "2", "--blockwise", "--pattern", "11110000", "--size", "512", "--skip-stats")
    assert rc == 0, out
    assert "Kernel 29 (ESMM A+B Optimized V3 (K26 + templated smem + float2 A-loads)): PASSED" in out
    assert "Kernel 15 (cuBLAS): PASSED" in out and "Summary: 2/2 kernels passed" in out
    assert "=== Skip Stats: K29 ===" in out and out.count("Kernel time:") == 2
    rc, out = run_ref("all", "1", "--size", "256", "--pattern", "11110000")
    assert rc == 0 and "Summary: 12/12 kernels passed" in out, out          # every id of the reference's switch
    rc, out = run_ref("20-30", "1", "--size", "256", "--random", "--no-check", "--verbose")
    assert rc == 0 and "Sparsity mode: RANDOM (unstructured)" in out and "Summary: 8/8 kernels completed (no verification)" in out
