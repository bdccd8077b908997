"""CPU tests of the drop-in surface: the reference's own driver.cu compiles, links and runs against this
repository's include/ (utils.cuh + runners.cuh) and libesmm_b200; the rand()-based generators exported
by the library reproduce the reference's matrices bit for bit (fixtures written by the reference's own
functions, tests/golden/make_golden.py); PatternLUT equals the reference's literal table."""
import ctypes as C
import os
import shutil
import subprocess

import numpy as np
import pytest

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")


@pytest.fixture(scope="module")
def ref_cpu():
    return np.load(os.path.join(GOLD, "ref_cpu.npz"))


@pytest.fixture(scope="module")
def gen(pkg):
    """The library's generator entry points with numpy arrays as arguments (host pointers)."""
    L = pkg.lib()

    class G:
        pass
    g = G()
    for name in ("with_pattern", "unstructured", "a_blocklevel", "b_blocklevel"):
        fn = getattr(L, "esmm_randomize_matrix_" + name)
        setattr(g, "esmm_randomize_matrix_" + name,
                lambda mat, *rest, _fn=fn: _fn(mat.ctypes.data if mat is not None else None, *rest))
    return g


def same_bits(a, b):
    return a.shape == b.shape and np.array_equal(a.view(np.uint32), b.view(np.uint32))


# ---- generators (include/utils.cuh:142-194, 303-426) -------------------------------------------------
def test_blockwise_generators_match_reference_bits(gen, ref_cpu):
    """--blockwise with the driver's seeds 12345 / 12346 (driver.cu:385,389)."""
    A = np.zeros((64, 64), np.float32)
    B = np.zeros((64, 128), np.float32)
    assert gen.esmm_randomize_matrix_a_blocklevel(A, 64, 64, 8, 32, 50.0, 12345) == 0
    assert gen.esmm_randomize_matrix_b_blocklevel(B, 64, 128, 8, 32, 50.0, 12346) == 0
    assert same_bits(A, ref_cpu["blk_A"]) and same_bits(B, ref_cpu["blk_B"])
    A8 = np.zeros((64, 64), np.float32)
    assert gen.esmm_randomize_matrix_a_blocklevel(A8, 64, 64, 8, 8, 75.0, 12345) == 0   # randomize_matrix_A<8,8>
    assert same_bits(A8, ref_cpu["a8_A"])


def test_default_pattern_generator_matches_reference_bits(gen, ref_cpu):
    """Default mode (driver.cu:403-406): no seeding of its own, A then B from one rand() stream; the sign is kept
    on an even draw and the fraction is scaled in double (include/utils.cuh:148-149)."""
    libc = C.CDLL(None)
    libc.srand(1)
    A = np.zeros((32, 64), np.float32)
    B = np.zeros((64, 32), np.float32)
    assert gen.esmm_randomize_matrix_with_pattern(A, 32, 64, b"11110000") == 0
    assert gen.esmm_randomize_matrix_with_pattern(B, 64, 32, b"11110000") == 0
    assert same_bits(A, ref_cpu["pat_A"]) and same_bits(B, ref_cpu["pat_B"])
    assert gen.esmm_randomize_matrix_with_pattern(A, 32, 64, b"1111") == 2      # ESMM_ERR_SHAPE
    assert gen.esmm_randomize_matrix_with_pattern(None, 32, 64, b"11110000") == 1    # ESMM_ERR_NULL


def test_unstructured_generator_matches_reference_bits(gen, ref_cpu):
    """--random (driver.cu:401-402): 37.5 % unstructured, seeds 12345 / 12346."""
    A = np.zeros((48, 40), np.float32)
    B = np.zeros((40, 56), np.float32)
    assert gen.esmm_randomize_matrix_unstructured(A, 48, 40, 37.5, 12345) == 0
    assert gen.esmm_randomize_matrix_unstructured(B, 40, 56, 37.5, 12346) == 0
    assert same_bits(A, ref_cpu["rnd_A"]) and same_bits(B, ref_cpu["rnd_B"])


# ---- PatternLUT (include/pattern_lut.cuh) ---------------------------------------------------------------
def test_pattern_lut_equals_reference_table(pkg, oracle_mod, ref_cpu):
    """All 256 entries of the reference's literal table (parsed from its header into the fixture) equal what the
    library and the oracle derive from the byte."""
    cnt_ref, off_ref = ref_cpu["lut_count"], ref_cpu["lut_offsets"]
    assert cnt_ref.shape == (256,) and off_ref.shape == (256, 8)
    L = pkg.lib()
    for p in range(256):
        cnt = C.c_uint8(0)
        off = (C.c_uint8 * 8)()
        L.esmm_pattern_lut(p, C.byref(cnt), C.byref(off))
        assert int(cnt.value) == int(cnt_ref[p]) and list(off) == list(off_ref[p]), p
        assert oracle_mod.pattern_lut(p) == (int(cnt_ref[p]), list(off_ref[p])), p


def test_pattern_lut_fixture_is_the_reference_header(oracle_mod, ref_cpu):
    """With the reference tree at hand, the fixture is re-derived from include/pattern_lut.cuh itself."""
    if not oracle_mod.have_ref_tree():
        pytest.skip("reference tree not present")
    from golden.make_golden import parse_pattern_lut
    cnt, off = parse_pattern_lut(os.path.join(oracle_mod.ref_root(), "include", "pattern_lut.cuh"))
    assert np.array_equal(cnt, ref_cpu["lut_count"]) and np.array_equal(off, ref_cpu["lut_offsets"])


# ---- the header swap ------------------------------------------------------------------------------------
def test_reference_driver_builds_against_this_include(pkg, oracle_mod, tmp_path):
    """The reference's driver.cu, byte for byte, placed in a directory without an include/ of its own and compiled
    with this repository's root on the include path: its `#include "include/utils.cuh"` and
    `#include "include/runners.cuh"` (driver.cu:1-2) then resolve to the headers here.  It must compile, link
    against libesmm_b200 + cuBLAS (driver.cu:419-442 calls cublasSgemm itself), and its argument handling must
    behave as the reference's (driver.cu:169-283)."""
    if not oracle_mod.have_ref_tree():
        pytest.skip("reference tree not present")
    if not os.path.exists(NVCC):
        pytest.skip("nvcc not present")
    src = tmp_path / "driver.cu"
    shutil.copyfile(os.path.join(oracle_mod.ref_root(), "driver.cu"), src)
    exe = tmp_path / "exec_swapped"
    lib_dir = os.path.dirname(pkg.LIB_PATH)
    cmd = [NVCC, "-O1", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a",
           "-I" + ROOT, str(src), "-o", str(exe), "-L" + lib_dir, "-lesmm_b200", "-lcublas",
           "-Xlinker", "-rpath", "-Xlinker", lib_dir]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stdout + p.stderr

    def run(*args):
        q = subprocess.run([str(exe), *args], capture_output=True, text=True, timeout=120)
        return q.returncode, q.stdout + q.stderr
    rc, out = run("--help")
    assert rc == 0 and "Usage:" in out and "--blockwise" in out and "29:" in out and "--gpus" not in out
    rc, out = run("99", "1")
    assert rc == 1 and "Error: Invalid kernel selection '99'" in out and "Usage:" in out
    rc, out = run("29", "1", "--pattern", "1100")
    assert rc == 1 and "Pattern must be exactly 8 characters" in out
    rc, out = run("29", "1", "--load-b", "w.bin")
    assert rc == 1 and "--dims M K N required with --load-a / --load-b" in out
