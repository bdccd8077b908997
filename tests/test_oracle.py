"""CPU tests of the oracle: pinned against the golden fixtures made from the unmodified reference
(tests/golden/make_golden.py) and against the closed-form expectations of the synthetic configs."""
import os

import numpy as np
import pytest

import workloads

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.fixture(scope="module")
def ref_cpu():
    return np.load(os.path.join(GOLD, "ref_cpu.npz"))


@pytest.fixture(scope="module")
def ref_gpu():
    return np.load(os.path.join(GOLD, "ref_gpu.npz"))


# ---- pins against the reference's own host code ---------------------------------------------
def test_cpu_sgemm_matches_reference_bits(oracle_mod, ref_cpu):
    """oracle.sgemm_naive restates matrixMultiplyCPU (include/utils.cuh:208-219): same bits."""
    for p in ("blk", "pat"):
        A, B, C = ref_cpu[p + "_A"], ref_cpu[p + "_B"], ref_cpu[p + "_C"]
        assert np.array_equal(oracle_mod.sgemm_naive(A, B), C)
        assert np.array_equal(oracle_mod.sgemm_naive(A, B, threads=3), C)
        assert np.array_equal(oracle_mod.sgemm_naive(A, B, rows=(8, 24)), C[8:24])


def test_reference_generator_block_structure(oracle_mod, ref_cpu):
    """Inputs drawn by the reference's --blockwise generators are block sparse at (32 x 8) / (8 x 32):
    every tile column / row is either all zero or (almost surely) not, and the oracle's patterns
    reproduce exactly the zero structure."""
    A, B = ref_cpu["blk_A"], ref_cpu["blk_B"]
    ap, bp = oracle_mod.preprocess_a(A), oracle_mod.preprocess_b(B)
    nzA = (A.reshape(2, 32, 8, 8) != 0).any(axis=1)   # [mb, kb, k]
    assert np.array_equal(np.packbits(nzA, axis=-1, bitorder="little")[..., 0], ap)
    nzB = (B.reshape(8, 8, 4, 32) != 0).any(axis=3)   # [kb, k, nb]
    assert np.array_equal(np.packbits(nzB.transpose(2, 0, 1), axis=-1, bitorder="little")[..., 0], bp)
    # the joint GEMM equals the dense CPU SGEMM up to float rounding (skipped terms are exact zeros)
    C = oracle_mod.gemm_joint(A, B, ap, bp)
    assert oracle_mod.rel_inf_err(C, ref_cpu["blk_C"]) <= 1e-5


def test_default_pattern_mode_masks_columns(oracle_mod, ref_cpu):
    """Default driver mode applies the pattern to the column index of whatever matrix it is given
    (include/utils.cuh:146): for A that is K, so the A pattern bytes are 0x0F for "11110000"."""
    ap = oracle_mod.preprocess_a(ref_cpu["pat_A"])
    assert set(ap.ravel()) <= {0x0F}


def test_oracle_matches_reference_gpu_kernels(oracle_mod, ref_gpu):
    """Pattern bytes of the reference's preprocess_ab<8,32,32> and C of its kernel id 29, captured
    on a B200, equal the oracle's bit for bit."""
    from golden.make_golden import GPU_CASES, make_case
    for name, M, N, K, gen, args in GPU_CASES:
        A, B = make_case(gen, M, N, K, args)
        ap, bp = oracle_mod.preprocess_a(A), oracle_mod.preprocess_b(B)
        assert np.array_equal(ap, ref_gpu[name + ".a_pat"]), name
        assert np.array_equal(bp, ref_gpu[name + ".b_pat"]), name
        if name + ".C" in ref_gpu:
            assert np.array_equal(oracle_mod.gemm_joint(A, B, ap, bp), ref_gpu[name + ".C"]), name


# ---- semantics --------------------------------------------------------------------------------
def test_pattern_string_and_lut(oracle_mod):
    assert [oracle_mod.pattern_from_string(s) for s in ("11111111", "11110000", "11000000", "10000000")] == \
        [0xFF, 0x0F, 0x03, 0x01]
    for bad in ("1111000", "111100000", "1111000x", ""):
        assert oracle_mod.pattern_from_string(bad) == -1
    for p in range(256):
        cnt, off = oracle_mod.pattern_lut(p)
        bits = [b for b in range(8) if p >> b & 1]
        assert cnt == len(bits) and off[:cnt] == bits and off[cnt:] == [0] * (8 - cnt)


def test_pattern_bit_order_and_index_order(oracle_mod):
    A = np.zeros((64, 32), np.float32)
    A[40, 19] = 1.0                       # row block 1, K block 2, k 3
    ap = oracle_mod.preprocess_a(A)
    assert ap.shape == (2, 4) and ap[1, 2] == 1 << 3 and ap.sum() == 8
    B = np.zeros((32, 96), np.float32)
    B[21, 70] = -2.0                      # K block 2, k 5, column block 2
    bp = oracle_mod.preprocess_b(B)
    assert bp.shape == (3, 4) and bp[2, 2] == 1 << 5 and bp.sum() == 32


def test_zero_tests(oracle_mod):
    A = np.zeros((32, 8), np.float32)
    A[0, 0] = -0.0
    A[1, 1] = np.nan
    A[2, 2] = np.float32(1e-45)           # denormal
    A[3, 3] = np.inf
    assert oracle_mod.preprocess_a(A)[0, 0] == 0b1110


def test_ragged_shapes(oracle_mod):
    rng = np.random.default_rng(3)
    A = rng.standard_normal((45, 20), dtype=np.float32)
    ap = oracle_mod.preprocess_a(A)
    assert ap.shape == (2, 3) and ap[1, 2] == 0x0F and ap[0, 0] == 0xFF
    ap8 = oracle_mod.preprocess_a(A, tile_m=8)
    assert ap8.shape == (6, 3)


def test_joint_gemm_vs_float64(oracle_mod):
    for (M, N, K, pa, pb, seed) in [(64, 128, 8, 1.0, 1.0, 0), (64, 128, 64, 0.5, 0.5, 1), (128, 256, 64, 0.2, 0.4, 2),
                                    (100, 132, 72, 0.6, 0.6, 3)]:
        A, B = workloads.tile_random(M, N, K, pa, pb, seed, gran_a=32, gran_b=32)
        C = oracle_mod.gemm_joint(A, B)
        assert oracle_mod.rel_inf_err(C, oracle_mod.sgemm_f64(A, B)) <= 1e-5
        # dropping terms whose joint bit is clear changes nothing: all of them are exact zeros
        assert oracle_mod.rel_inf_err(C, oracle_mod.sgemm_naive(A, B)) <= 1e-5


def test_verify_results_semantics(oracle_mod):
    ref = np.zeros(10, np.float32)
    gpu = ref.copy()
    gpu[3] = 0.02
    gpu[7] = -0.5
    gpu[8] = 0.009
    bad, maxd, first = oracle_mod.verify_results(gpu, ref, 1e-2)
    assert (bad, first) == (2, 3) and maxd == pytest.approx(0.5)


# ---- closed-form expectations of the synthetic configs ---------------------------------------------
@pytest.mark.parametrize("pat,density", [(0xFF, 1.0), (0x0F, 0.5), (0x03, 0.25), (0x01, 0.125)])
def test_uniform_pattern_stats(oracle_mod, pat, density):
    M = N = K = 256
    A, B = workloads.uniform_pattern(M, N, K, pat, seed=0)
    ap, bp = oracle_mod.preprocess_a(A), oracle_mod.preprocess_b(B)
    assert set(ap.ravel()) == {pat} and set(bp.ravel()) == {pat}
    st = oracle_mod.skip_stats(ap, bp, 2, 4)
    assert st["block_skips"] == 0 and st["warp_skips"] == 0
    assert st["total_dot"] - st["dot_skips"] == int(density * st["total_dot"])
    assert oracle_mod.executed_macs(ap, bp) == int(density * M * N * K)


def test_tile_random_stats(oracle_mod):
    M = N = 1024
    K = 2048
    A, B = workloads.tile_random(M, N, K, 0.5, 0.5, seed=1)
    ap, bp = oracle_mod.preprocess_a(A), oracle_mod.preprocess_b(B)
    assert np.array_equal(ap[0::2], ap[1::2]) and np.array_equal(bp[0::2], bp[1::2])  # generator granularity 64
    st = oracle_mod.skip_stats(ap, bp, 2, 4)
    assert oracle_mod.executed_macs(ap, bp) / (M * N * K) == pytest.approx(0.25, abs=0.01)
    assert st["warp_skips"] / st["total_warp_k"] == pytest.approx(0.75 ** 8, abs=0.01)
    assert st["block_skips"] / st["total_k"] == pytest.approx(0.625 ** 8, abs=0.01)


def test_llm_mlp_workload(oracle_mod):
    A, B = workloads.llm_mlp(256, 512, 1024, seed=0)
    ap, bp = oracle_mod.preprocess_a(A), oracle_mod.preprocess_b(B)
    assert (ap == 0).mean() == pytest.approx(0.6, abs=0.02)
    assert (bp == 0).mean() == pytest.approx(0.5, abs=0.02)
    assert set(bp.ravel()) <= {0, 0xFF}
    assert np.array_equal(bp[0::2], bp[1::2])


def test_all_byte_values_workload(oracle_mod):
    A, B = workloads.all_byte_values(64, 128)
    ap, bp = oracle_mod.preprocess_a(A), oracle_mod.preprocess_b(B)
    assert set(ap.ravel()) == set(range(256)) and set(bp.ravel()) == set(range(256))
