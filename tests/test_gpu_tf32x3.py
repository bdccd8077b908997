"""GPU tests of the optional 3xTF32 tensor-core entry point (esmm_sgemm_joint_tf32x3) against the CPU oracle.

This variant is not bit-identical to the FP32 FMA chain: the bound checked is the path's own tolerance,
max |C - C_oracle| / max |C_oracle| <= 1e-4, and, tighter, the 1e-5 that its run-wise accumulation is built to
keep at every K tested here.  Where a product is exactly zero (dead tiles) the result must be exactly zero."""
import numpy as np
import pytest

import workloads

pytestmark = pytest.mark.gpu
TOL = 1e-4      # the tolerance of the path's specification
TIGHT = 1e-5    # what 3xTF32 with 256-k accumulation runs delivers in practice


def run_tf32x3(torch, pkg, A, B, compact=True, calls=1):
    M, K = A.shape
    N = B.shape[1]
    dA = torch.from_numpy(np.ascontiguousarray(A)).cuda()
    dB = torch.from_numpy(np.ascontiguousarray(B)).cuda()
    b = pkg.Tf32x3B(dB.data_ptr(), K, N, compact)
    ws = torch.empty(pkg.tf32x3_workspace_bytes(M, K), dtype=torch.uint8, device="cuda")
    ws.fill_(0xFF)                                   # NaN bit patterns wherever the split does not write
    out = []
    for _ in range(calls):
        c = torch.full((M, N), float("nan"), device="cuda")
        pkg.sgemm_joint_tf32x3(M, dA.data_ptr(), b, c.data_ptr(), ws.data_ptr())
        pkg.device_status()
        out.append(c.cpu().numpy())
    live_k = b.live_k
    b.close()
    return out if calls > 1 else out[0], live_k


def rel_inf(c, ref):
    scale = float(np.abs(ref).max())
    return float(np.abs(c.astype(np.float64) - ref.astype(np.float64)).max()) / (scale if scale > 0 else 1.0)


@pytest.mark.parametrize("pat", ["11111111", "11110000", "11000000", "10000000", "10100101", "00000001"])
@pytest.mark.parametrize("compact", [True, False])
def test_uniform_patterns(cuda, pkg, oracle_mod, pat, compact):
    M, N, K = 256, 384, 1024
    byte = workloads.pattern_byte(pat)
    A, B = workloads.uniform_pattern(M, N, K, byte, seed=11)
    c, live_k = run_tf32x3(cuda, pkg, A, B, compact)
    ref = oracle_mod.gemm_joint(A, B)
    assert not np.isnan(c).any()
    assert rel_inf(c, ref) <= TIGHT <= TOL
    kept = K * bin(byte).count("1") // 8
    assert live_k == (kept if compact and kept < K else K)      # 1024 * popcount / 8 is a multiple of 32 here


@pytest.mark.parametrize("M,N,K,pa,pb", [
    (128, 128, 8, 1.0, 1.0),          # one tile, one K block: the fetch box is wider than the matrix
    (96, 132, 24, 0.7, 0.7),          # ragged M and N, K below one fetch group
    (200, 260, 136, 0.5, 0.5),        # ragged everything, K % 32 != 0
    (512, 640, 2048, 0.3, 0.3),
    (1024, 1024, 1024, 0.05, 0.05),   # many dead K blocks and dead tiles
    (32, 4096, 512, 0.5, 0.5),        # one row block of A
])
def test_tile_random(cuda, pkg, oracle_mod, M, N, K, pa, pb):
    A, B = workloads.tile_random(M, N, K, pa, pb, seed=5, gran_a=32, gran_b=32)
    c, _ = run_tf32x3(cuda, pkg, A, B)
    assert rel_inf(c, oracle_mod.gemm_joint(A, B)) <= TIGHT


@pytest.mark.parametrize("pair", ["0", "128", "256"])
def test_kernel_variants_agree(cuda, pkg, oracle_mod, tuning, pair):
    """ESMM_TF32_PAIR selects the kernel: 0 = one CTA per 128 x 128 tile, 128 / 256 = a CTA pair (cta_group::2) per
    256 x 128 / 256 x 256 tile (the default where M and N allow).  Ragged sizes, dead K blocks, several tiles per CTA."""
    tuning("TF32_PAIR", int(pair))
    for (M, N, K, pa, pb, seed) in [(520, 776, 1032, 0.2, 0.2, 1), (256, 256, 64, 1.0, 1.0, 2), (2048, 2304, 512, 0.5, 0.5, 3)]:
        A, B = workloads.tile_random(M, N, K, pa, pb, seed=seed, gran_a=32, gran_b=32)
        A[300:460] = 0.0                     # a dead band of A: tiles and half-tiles without work
        c, _ = run_tf32x3(cuda, pkg, A, B)
        assert rel_inf(c, oracle_mod.gemm_joint(A, B)) <= TIGHT, (M, N, K)
        assert not c[300:460].any()


@pytest.mark.parametrize("compact", [True, False])
def test_block_structured_and_dead_tiles(cuda, pkg, oracle_mod, compact):
    """Whole pattern blocks dead (K-block skipping does all the work), plus a band of A and a band of B that
    are zero altogether: those tiles of C never see an MMA and must come out as exact zeros."""
    M, N, K = 512, 512, 1024
    A, B = workloads.block_random(M, N, K, 0.3, 0.3, seed=2)
    A[128:256] = 0.0
    B[:, 256:384] = 0.0
    c, _ = run_tf32x3(cuda, pkg, A, B, compact)
    assert rel_inf(c, oracle_mod.gemm_joint(A, B)) <= TIGHT
    assert not c[128:256].any() and not c[:, 256:384].any()


def test_dead_rows_of_b_are_dropped_and_padded(cuda, pkg, oracle_mod):
    """Rows of B zeroed at random: the kept k are no multiple of 32, so the list is padded with zero columns."""
    M, N, K = 160, 256, 512
    rng = np.random.default_rng(4)
    A = rng.standard_normal((M, K), dtype=np.float32)
    B = rng.standard_normal((K, N), dtype=np.float32)
    dead = rng.random(K) < 0.6
    B[dead] = 0.0
    c, live_k = run_tf32x3(cuda, pkg, A, B, compact=True)
    kept = int((~dead).sum())
    assert live_k == -(-kept // 32) * 32 and live_k < K
    assert rel_inf(c, oracle_mod.gemm_joint(A, B)) <= TIGHT
    c2, k2 = run_tf32x3(cuda, pkg, A, B, compact=False)
    assert k2 == K and rel_inf(c2, oracle_mod.gemm_joint(A, B)) <= TIGHT


def test_all_zero_operands(cuda, pkg):
    M, N, K = 128, 256, 64
    rng = np.random.default_rng(0)
    Z = np.zeros((K, N), dtype=np.float32)
    A = rng.standard_normal((M, K), dtype=np.float32)
    c, live_k = run_tf32x3(cuda, pkg, A, Z)
    assert live_k == 32 and not c.any()
    c, _ = run_tf32x3(cuda, pkg, np.zeros((M, K), dtype=np.float32), rng.standard_normal((K, N), dtype=np.float32))
    assert not c.any()


def test_wide_dynamic_range_and_repeatability(cuda, pkg, oracle_mod):
    """Values over twelve orders of magnitude (the split must hold the low part of large and of tiny values);
    two calls in a row on the same handle and workspace give the same bits."""
    M, N, K = 256, 256, 768
    rng = np.random.default_rng(8)
    A = (rng.standard_normal((M, K)) * np.exp(rng.uniform(-14, 14, (M, K)))).astype(np.float32)
    B = (rng.standard_normal((K, N)) * np.exp(rng.uniform(-14, 14, (K, N)))).astype(np.float32)
    (c1, c2), _ = run_tf32x3(cuda, pkg, A, B, calls=2)
    assert np.array_equal(c1, c2)
    assert rel_inf(c1, oracle_mod.gemm_joint(A, B)) <= TIGHT


def test_long_k_accuracy_against_float64(cuda, pkg):
    """K = 16384 (the multi-GPU configuration's depth): the error against the exact product stays at the level
    of an FP32 FMA chain instead of growing with K as a single tensor-core accumulation would."""
    for M, N in ((128, 256), (256, 512)):      # one CTA per tile; CTA pairs
        K = 16384
        A, B = workloads.uniform_pattern(M, N, K, 0xFF, seed=21)
        c, _ = run_tf32x3(cuda, pkg, A, B)
        ref = A.astype(np.float64) @ B.astype(np.float64)
        assert rel_inf(c, ref) <= TIGHT, (M, N)


def test_full_size_agrees_with_fp32_path(cuda, pkg):
    """4096^3 at 50 % (pattern 11110000): the tensor-core result against the FP32 joint-sparse path on the
    device (itself bit-identical to the oracle at the sizes the oracle can run)."""
    torch = cuda
    M = N = K = 4096
    A, B = workloads.uniform_pattern(M, N, K, 0x0F, seed=3)
    c, live_k = run_tf32x3(torch, pkg, A, B)
    assert live_k == K // 2
    dA, dB = torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda()
    bp = torch.empty((N // 32, K // 8), dtype=torch.uint8, device="cuda")
    pkg.preprocess_b(dB.data_ptr(), K, N, bp.data_ptr())
    ws = torch.empty(pkg.sgemm_joint_workspace_bytes(M, K), dtype=torch.uint8, device="cuda")
    ref = torch.empty((M, N), device="cuda")
    pkg.sgemm_joint(M, N, K, dA.data_ptr(), dB.data_ptr(), ref.data_ptr(), bp.data_ptr(), ws.data_ptr())
    pkg.device_status()
    assert rel_inf(c, ref.cpu().numpy()) <= TIGHT


@pytest.mark.parametrize("pair", ["256", "128"])
def test_last_round_split_along_k(cuda, pkg, tuning, pair):
    """Shapes whose tiles leave a partly filled last wave: those tiles are computed as two halves of K by two CTA
    pairs that add into a zeroed C.  Same result as without the split to rounding, the same bits on every call,
    and stale contents of C do not leak in."""
    torch = cuda
    tuning("TF32_PAIR", int(pair))
    M, N, K = (2560, 2560, 2048) if pair == "256" else (2560, 1280, 2048)     # 100 tiles for 74 pairs: 26 are split
    A, B = workloads.tile_random(M, N, K, 0.6, 0.6, seed=12, gran_a=32, gran_b=32)
    A[:, 1024:1536] = 0.0                                                     # dead groups in the middle of K
    dA, dB = torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda()
    bp = torch.empty((N // 32, K // 8), dtype=torch.uint8, device="cuda")
    pkg.preprocess_b(dB.data_ptr(), K, N, bp.data_ptr())
    ws = torch.empty(pkg.sgemm_joint_workspace_bytes(M, K), dtype=torch.uint8, device="cuda")
    ref = torch.empty((M, N), device="cuda")
    pkg.sgemm_joint(M, N, K, dA.data_ptr(), dB.data_ptr(), ref.data_ptr(), bp.data_ptr(), ws.data_ptr())
    pkg.device_status()
    ref = ref.cpu().numpy()
    (c1, c2), _ = run_tf32x3(torch, pkg, A, B, calls=2)                        # C starts as NaN in both calls
    assert np.array_equal(c1, c2)
    assert rel_inf(c1, ref) <= TIGHT
    tuning("TF32_SPLIT_LAST", 0)
    c3, _ = run_tf32x3(torch, pkg, A, B)
    assert rel_inf(c3, ref) <= TIGHT and rel_inf(c1, c3) <= TIGHT


def test_argument_checks(cuda, pkg):
    import ctypes as C
    torch = cuda
    L = pkg.lib()
    B = torch.zeros((64, 128), device="cuda")
    h = C.c_void_p()
    assert L.esmm_tf32x3_b_create(None, 64, 128, 1, C.byref(h)) == 1            # ESMM_ERR_NULL
    assert L.esmm_tf32x3_b_create(B.data_ptr(), 60, 128, 1, C.byref(h)) == 2     # K % 8
    assert L.esmm_tf32x3_b_create(B.data_ptr(), 64, 126, 1, C.byref(h)) == 2     # N % 4
    assert L.esmm_tf32x3_b_create(B.data_ptr() + 4, 64, 128, 1, C.byref(h)) == 3  # alignment
    assert not h.value
    b = pkg.Tf32x3B(B.data_ptr(), 64, 128)
    ws = torch.empty(pkg.tf32x3_workspace_bytes(32, 64) + 256, dtype=torch.uint8, device="cuda")
    A = torch.zeros((32, 64), device="cuda")
    c = torch.zeros((32, 128), device="cuda")
    assert L.esmm_sgemm_joint_tf32x3(32, A.data_ptr(), b.handle, c.data_ptr(), None, None) == 1
    assert L.esmm_sgemm_joint_tf32x3(0, A.data_ptr(), b.handle, c.data_ptr(), ws.data_ptr(), None) == 2
    assert L.esmm_sgemm_joint_tf32x3(32, A.data_ptr(), b.handle, c.data_ptr(), ws.data_ptr() + 16, None) == 3
    L.esmm_tf32x3_b_destroy(None)                                              # a no-op
    b.close()


def test_runner_id_129_and_cli(cuda, pkg, oracle_mod, capfd):
    """The reference's timed runner loop (verification against the cuBLAS result included) with the tensor-core
    variant as additive kernel id 129, through the C ABI and through the exec_b200 command line."""
    import ctypes as C
    import subprocess
    M = N = K = 512
    A, B = workloads.tile_random(M, N, K, 0.5, 0.5, seed=31, gran_a=64, gran_b=32)
    dA, dB = cuda.from_numpy(A).cuda(), cuda.from_numpy(B).cuda()
    dC = cuda.zeros((M, N), device="cuda")
    h_ref, h_c = np.zeros((M, N), np.float32), np.zeros((M, N), np.float32)
    L = pkg.lib()
    passed, avg = C.c_int(0), C.c_float(0)
    assert L.esmm_run_kernel(15, M, N, K, dA.data_ptr(), dB.data_ptr(), dC.data_ptr(), h_ref.ctypes.data, None, 1, 0,
                             0, C.byref(passed), C.byref(avg)) == 0
    st = L.esmm_run_kernel(129, M, N, K, dA.data_ptr(), dB.data_ptr(), dC.data_ptr(), h_c.ctypes.data,
                           h_ref.ctypes.data, 3, 1, 1, C.byref(passed), C.byref(avg))
    assert st == 0 and passed.value == 1 and avg.value > 0
    assert rel_inf(h_c, oracle_mod.gemm_joint(A, B)) <= TIGHT
    out = capfd.readouterr().out
    assert "=== Skip Stats: K129 ===" in out
    # K not a multiple of 8 is outside what the tensor-core path takes: a status, no launch
    st = L.esmm_run_kernel(129, 64, 64, 60, dA.data_ptr(), dB.data_ptr(), dC.data_ptr(), h_c.ctypes.data,
                           h_ref.ctypes.data, 1, 0, 0, C.byref(passed), C.byref(avg))
    assert st == 2
    p = subprocess.run([pkg.EXE_PATH, "129", "2", "--size", "512", "--pattern", "11110000"], capture_output=True,
                       text=True, timeout=600)
    assert p.returncode == 0 and "PASSED" in p.stdout.upper(), p.stdout + p.stderr
