"""GPU parity tests: every compute entry point of the C ABI against the CPU oracle (bit-exact for
pattern bytes; C within rel-inf 1e-4, and in practice bit-identical), against the golden outputs of
the reference's own GPU kernels, and - at the benchmark's full sizes - through size-independent
properties."""
import ctypes as C
import os

import numpy as np
import pytest

import workloads

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
TOL = 1e-4  # max |C - C_ref| / max |C_ref|, the tolerance of the path's specification


class Dev:
    """Device buffers for one problem, through torch (plumbing only)."""

    def __init__(self, torch, pkg, A, B):
        self.torch, self.pkg = torch, pkg
        self.M, self.K = A.shape
        self.N = B.shape[1]
        self.A = torch.from_numpy(np.ascontiguousarray(A)).cuda()
        self.B = torch.from_numpy(np.ascontiguousarray(B)).cuda()
        self.nKB = -(-self.K // 8)
        self.ap = torch.full((-(-self.M // 32), self.nKB), 0xEE, dtype=torch.uint8, device="cuda")
        self.bp = torch.full((-(-self.N // 32), self.nKB), 0xEE, dtype=torch.uint8, device="cuda")

    def C(self):
        return self.torch.full((self.M, self.N), float("nan"), device="cuda")

    def patterns(self):
        self.pkg.preprocess_a(self.A.data_ptr(), self.M, self.K, self.ap.data_ptr())
        self.pkg.preprocess_b(self.B.data_ptr(), self.K, self.N, self.bp.data_ptr())
        self.torch.cuda.synchronize()
        return self.ap.cpu().numpy(), self.bp.cpu().numpy()

    def gemm_rowmajor(self):
        c = self.C()
        self.pkg.gemm_ab(self.M, self.N, self.K, self.A.data_ptr(), self.B.data_ptr(), c.data_ptr(),
                         self.ap.data_ptr(), self.bp.data_ptr())
        self.pkg.device_status()
        return c.cpu().numpy()

    def sgemm_joint(self, poison=True):
        """The per-call path: packing preprocess + packed GEMM; returns (C, A patterns it wrote)."""
        c = self.C()
        ws = self.torch.empty(self.pkg.sgemm_joint_workspace_bytes(self.M, self.K), dtype=self.torch.uint8,
                              device="cuda")
        if poison:
            ws.fill_(0xFF)  # entries the packer leaves unwritten hold NaN bit patterns
        self.pkg.sgemm_joint(self.M, self.N, self.K, self.A.data_ptr(), self.B.data_ptr(), c.data_ptr(),
                             self.bp.data_ptr(), ws.data_ptr())
        self.pkg.device_status()
        n = self.ap.numel()
        return c.cpu().numpy(), ws[:n].reshape(self.ap.shape).cpu().numpy()


def check_all_paths(cuda, pkg, oracle_mod, A, B, expect_bits=True):
    d = Dev(cuda, pkg, A, B)
    ap, bp = d.patterns()
    oap, obp = oracle_mod.preprocess_a(A), oracle_mod.preprocess_b(B)
    assert np.array_equal(ap, oap), "A pattern bytes differ from the oracle"
    assert np.array_equal(bp, obp), "B pattern bytes differ from the oracle"
    Cref = oracle_mod.gemm_joint(A, B, oap, obp)
    C1 = d.gemm_rowmajor()
    C2, ap2 = d.sgemm_joint()
    assert np.array_equal(ap2, oap), "packing preprocessor: A pattern bytes differ from the oracle"
    for name, Cg in (("row-major kernel", C1), ("packed kernel", C2)):
        assert not np.isnan(Cg).any(), name
        assert oracle_mod.rel_inf_err(Cg, Cref) <= TOL, name
        if expect_bits:
            assert np.array_equal(Cg, Cref), f"{name}: not bit-identical to the oracle's FMA chain"
    return Cref


# ---- pattern preprocessor ------------------------------------------------------------------------
@pytest.mark.parametrize("M,K", [(32, 8), (64, 128), (1024, 1024), (100, 72), (16, 256), (33, 132), (257, 1000)])
def test_preprocess_a_shapes(cuda, pkg, oracle_mod, M, K):
    A, _ = workloads.tile_random(M, 32, K, 0.4, 1.0, seed=M + K, gran_a=32)
    dA = cuda.from_numpy(A).cuda()
    for tile_m in (32, 64, 8):
        out = cuda.full((-(-M // tile_m), -(-K // 8)), 0xEE, dtype=cuda.uint8, device="cuda")
        pkg.preprocess_a(dA.data_ptr(), M, K, out.data_ptr(), tile_m=tile_m)
        cuda.cuda.synchronize()
        assert np.array_equal(out.cpu().numpy(), oracle_mod.preprocess_a(A, tile_m)), (M, K, tile_m)


def test_preprocess_generic_kernels_for_unaligned_k(cuda, pkg, oracle_mod):
    """K or N not a multiple of 4 takes the one-thread-per-byte kernels."""
    rng = np.random.default_rng(5)
    A = rng.standard_normal((70, 30), dtype=np.float32) * (rng.random((70, 30)) < 0.1)
    B = rng.standard_normal((30, 70), dtype=np.float32) * (rng.random((30, 70)) < 0.1)
    dA, dB = cuda.from_numpy(A).cuda(), cuda.from_numpy(B).cuda()
    oa = cuda.zeros((3, 4), dtype=cuda.uint8, device="cuda")
    ob = cuda.zeros((3, 4), dtype=cuda.uint8, device="cuda")
    pkg.preprocess_a(dA.data_ptr(), 70, 30, oa.data_ptr())
    pkg.preprocess_b(dB.data_ptr(), 30, 70, ob.data_ptr())
    cuda.cuda.synchronize()
    assert np.array_equal(oa.cpu().numpy(), oracle_mod.preprocess_a(A))
    assert np.array_equal(ob.cpu().numpy(), oracle_mod.preprocess_b(B))


def test_preprocess_single_nonzero_at_every_position(cuda, pkg, oracle_mod):
    """One nonzero at each (row % 32, k % 8) position of A and (k % 8, col % 32) of B in turn."""
    M, K, N = 64, 128, 64
    for r in (0, 1, 15, 31, 32, 63):
        for k in range(8):
            A = np.zeros((M, K), np.float32)
            A[r, 40 + k] = 1.0
            B = np.zeros((K, N), np.float32)
            B[88 + k, r] = -1.0
            d = Dev(cuda, pkg, A, B)
            ap, bp = d.patterns()
            assert np.array_equal(ap, oracle_mod.preprocess_a(A)) and ap.sum() == 1 << k
            assert np.array_equal(bp, oracle_mod.preprocess_b(B)) and bp.sum() == 1 << k


def test_preprocess_zero_semantics(cuda, pkg, oracle_mod):
    A = np.zeros((32, 8), np.float32)
    A[0, 0] = -0.0
    A[1, 1] = np.nan
    A[2, 2] = np.float32(1e-45)
    A[3, 3] = np.inf
    B = np.ascontiguousarray(A.T)
    d = Dev(cuda, pkg, A, B)
    ap, bp = d.patterns()
    assert ap[0, 0] == 0b1110 and bp[0, 0] == 0b1110
    assert np.array_equal(ap, oracle_mod.preprocess_a(A))


def test_preprocess_ab_metadata(cuda, pkg, oracle_mod):
    A, B = workloads.tile_random(128, 256, 512, 0.5, 0.5, seed=9, gran_a=32, gran_b=32)
    dA, dB = cuda.from_numpy(A).cuda(), cuda.from_numpy(B).cuda()
    meta = pkg.ABPatternMetadata()
    pkg.check(pkg.lib().esmm_preprocess_ab(dA.data_ptr(), dB.data_ptr(), 128, 256, 512, 32, None, C.byref(meta)),
              "esmm_preprocess_ab")
    cuda.cuda.synchronize()
    assert (meta.numMBlocks, meta.numNBlocks, meta.numKBlocks, meta.owns_b_patterns) == (4, 8, 64, 1)
    ha = np.zeros((4, 64), np.uint8)
    hb = np.zeros((8, 64), np.uint8)
    rt = C.CDLL("libcudart.so.12")
    rt.cudaMemcpy.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_int]
    assert rt.cudaMemcpy(ha.ctypes.data, meta.d_a_patterns, ha.size, 2) == 0
    assert rt.cudaMemcpy(hb.ctypes.data, meta.d_b_patterns, hb.size, 2) == 0
    assert np.array_equal(ha, oracle_mod.preprocess_a(A)) and np.array_equal(hb, oracle_mod.preprocess_b(B))
    cached = meta.d_b_patterns
    meta2 = pkg.ABPatternMetadata()
    pkg.check(pkg.lib().esmm_preprocess_ab(dA.data_ptr(), None, 128, 256, 512, 32, cached, C.byref(meta2)),
              "esmm_preprocess_ab(cached)")
    assert meta2.owns_b_patterns == 0 and meta2.d_b_patterns == cached
    pkg.lib().esmm_free_ab_pattern_metadata(C.byref(meta2))
    pkg.lib().esmm_free_ab_pattern_metadata(C.byref(meta))
    assert meta.d_a_patterns is None and meta.d_b_patterns is None


# ---- joint-sparse GEMM: both kernels against the oracle ----------------------------------------------
@pytest.mark.parametrize("pat", [0xFF, 0x0F, 0x03, 0x01, 0xA5, 0x80, 0x3C])
def test_gemm_uniform_patterns(cuda, pkg, oracle_mod, tuning, pat):
    """Tiles whose K blocks all hold the same run of 1, 2, 4 or 8 consecutive live k need no row list (0xFF,
    0x0F, 0x03, 0x01, 0x80, 0x3C here); the same inputs with that shortcut switched off, and patterns that
    are no such run (0xA5), take the general listing."""
    A, B = workloads.uniform_pattern(256, 256, 512, pat, seed=pat)
    check_all_paths(cuda, pkg, oracle_mod, A, B)
    tuning("NO_RUN_TILES", 1)
    check_all_paths(cuda, pkg, oracle_mod, A, B)
    tuning.reset()
    # K blocks not a multiple of the stage depth (last stage partial) and a ragged edge tile
    A, B = workloads.uniform_pattern(200, 160, 8 * 21, pat, seed=pat + 1)
    check_all_paths(cuda, pkg, oracle_mod, A, B)


@pytest.mark.parametrize("M,N,K,pa,pb", [
    (128, 128, 8, 1.0, 1.0),        # one K block
    (128, 128, 16, 0.5, 0.5),
    (256, 384, 512, 0.5, 0.5),
    (512, 512, 1024, 0.2, 0.2),     # many dead K tiles
    (384, 256, 264, 0.3, 0.7),      # K blocks not a multiple of the stage depth
    (128, 256, 2048, 0.05, 0.9),
    (100, 132, 72, 0.6, 0.6),       # ragged M, N; K % 8 == 0
    (16, 256, 256, 0.5, 0.5),       # fewer rows than one pattern block
    (130, 64, 128, 0.7, 0.7),       # N smaller than one tile
    (64, 4, 64, 1.0, 1.0),          # minimal N
    (96, 160, 76, 0.8, 0.8),        # K % 8 == 4
])
def test_gemm_tile_random(cuda, pkg, oracle_mod, M, N, K, pa, pb):
    A, B = workloads.tile_random(M, N, K, pa, pb, seed=M + N + K, gran_a=32, gran_b=32)
    check_all_paths(cuda, pkg, oracle_mod, A, B)


def test_gemm_every_pattern_byte(cuda, pkg, oracle_mod):
    A, B = workloads.all_byte_values(128, 256, seed=1)
    check_all_paths(cuda, pkg, oracle_mod, A, B)


def test_gemm_all_zero_inputs(cuda, pkg, oracle_mod):
    A = np.zeros((128, 64), np.float32)
    B = np.random.default_rng(0).standard_normal((64, 128), dtype=np.float32)
    Cref = check_all_paths(cuda, pkg, oracle_mod, A, B)
    assert not Cref.any()


def test_gemm_llm_mlp_shapes(cuda, pkg, oracle_mod):
    """Config 4 at reduced width: activations (M = 16 and M = 256) x pruned weights."""
    for M in (16, 256):
        A, B = workloads.llm_mlp(M, 1408, 1024, seed=M)
        check_all_paths(cuda, pkg, oracle_mod, A, B)


def test_gemm_long_k_multi_tile_per_cta(cuda, pkg, oracle_mod, tuning):
    """2048 K blocks (the reference kernel stops at 1024) and several tiles per CTA."""
    tuning("GRID", 3)
    A, B = workloads.tile_random(256, 512, 16384, 0.15, 0.5, seed=4)
    check_all_paths(cuda, pkg, oracle_mod, A, B)


@pytest.mark.parametrize("stages", [2, 3])
def test_gemm_shallow_ring(cuda, pkg, oracle_mod, tuning, stages):
    tuning("STAGES", int(stages))
    A, B = workloads.tile_random(256, 256, 1024, 0.5, 0.5, seed=11)
    check_all_paths(cuda, pkg, oracle_mod, A, B)


@pytest.mark.parametrize("brow", [0, 1, 8])
def test_gemm_row_fetch_policies(cuda, pkg, oracle_mod, tuning, brow):
    tuning("BROW_BITS", int(brow))
    A, B = workloads.tile_random(256, 256, 512, 0.3, 0.4, seed=12, gran_a=32, gran_b=32)
    check_all_paths(cuda, pkg, oracle_mod, A, B)
    A, B = workloads.uniform_pattern(128, 128, 256, 0x03, seed=1)
    check_all_paths(cuda, pkg, oracle_mod, A, B)


@pytest.mark.parametrize("rows", [64, 128])
def test_gemm_both_tile_heights(cuda, pkg, oracle_mod, tuning, rows):
    """The packed kernel tiles C in 128 x 128 or, where that fills the GPU better, 64 x 128 (a 64-row tile is
    one half of a 128-row panel of packed A).  Both tilings, forced, on uniform, random, ragged and small-M
    inputs: same bits as the oracle."""
    tuning("TILE_M", int(rows))
    for pat in (0xFF, 0x0F, 0x01, 0x24):
        A, B = workloads.uniform_pattern(384, 256, 512, pat, seed=pat)
        check_all_paths(cuda, pkg, oracle_mod, A, B)
    A, B = workloads.tile_random(320, 384, 1024, 0.4, 0.5, seed=21, gran_a=32, gran_b=32)
    check_all_paths(cuda, pkg, oracle_mod, A, B)
    A, B = workloads.tile_random(200, 132, 250 * 4, 0.5, 0.5, seed=22, gran_a=32, gran_b=32)   # ragged M, N
    check_all_paths(cuda, pkg, oracle_mod, A, B)
    A, B = workloads.all_byte_values(seed=23)
    check_all_paths(cuda, pkg, oracle_mod, A, B)
    for M in (16, 48, 96):
        A, B = workloads.llm_mlp(M, 512, 1024, seed=M)
        check_all_paths(cuda, pkg, oracle_mod, A, B)
    tuning("FORCE_LISTED", 1)
    A, B = workloads.uniform_pattern(192, 256, 256, 0x0F, seed=2)
    check_all_paths(cuda, pkg, oracle_mod, A, B)


@pytest.mark.parametrize("producers", [7, 0, 3])
@pytest.mark.parametrize("rows", [128, 64])
def test_gemm_producer_warp_forms(cuda, pkg, oracle_mod, tuning, rows, producers):
    """The launch shapes of the tiled kernel, each pinned with esmm_tuning_set("PRODUCER_WARPS", v): 7 = the 16-warp
    form (registers moved between warp groups with setmaxnreg) with all 7 producer warps copying, 0 = the same form
    where each CTA's first tile decides between 3 and 7, 3 = the 12-warp form.  Run tiles, row-by-row stages, boxes
    of 1 / 2 / 4 / 8 consecutive rows, ragged edges, both tile heights - the same bits as the oracle in every shape."""
    tuning("PRODUCER_WARPS", int(producers))
    tuning("TILE_M", int(rows))
    for pat in (0xFF, 0x0F, 0x01):
        A, B = workloads.uniform_pattern(256, 384, 512, pat, seed=pat)
        check_all_paths(cuda, pkg, oracle_mod, A, B)
    for M, N, K, pa, pb, ga in [(512, 512, 1024, 0.2, 0.2, 32), (384, 256, 2048, 0.5, 0.5, 64), (257, 260, 1000, 0.4, 0.4, 32),
                                (100, 132, 8 * 37, 0.3, 0.7, 32), (256, 512, 8192 + 128, 0.3, 0.5, 32)]:
        A, B = workloads.tile_random(M, N, K, pa, pb, seed=M + K, gran_a=ga, gran_b=32)
        check_all_paths(cuda, pkg, oracle_mod, A, B)
    A, B = workloads.block_random(384, 512, 1024, 0.3, 0.4, seed=9)
    check_all_paths(cuda, pkg, oracle_mod, A, B)
    A, B = workloads.llm_mlp(256, 1408, 1024, seed=4)
    check_all_paths(cuda, pkg, oracle_mod, A, B)


@pytest.mark.parametrize("producers", [3, 0])
def test_gemm_boxes_of_consecutive_rows(cuda, pkg, oracle_mod, tuning, producers):
    """Listed rows with consecutive k are fetched in boxes of 8, 4, 2 and 1 rows.  Uniform patterns whose live k form
    runs of every length from 1 to 14 (0xE7: k 5, 6, 7 of one K block and 0, 1, 2 of the next are one run of 6), with
    K such that runs straddle stage boundaries and the last stage is ragged; both launch shapes."""
    tuning("PRODUCER_WARPS", int(producers))
    for pat in (0xE7, 0x7E, 0xDB, 0xFE, 0x7F, 0xBF, 0x55, 0x33, 0xF1, 0x9F):
        for M, N, K in ((256, 384, 512), (130, 132, 8 * 37)):
            A, B = workloads.uniform_pattern(M, N, K, pat, seed=pat)
            check_all_paths(cuda, pkg, oracle_mod, A, B)
    A, B = workloads.all_byte_values(M=256, N=256, seed=16)
    check_all_paths(cuda, pkg, oracle_mod, A, B)


def test_gemm_ordinary_launch(cuda, pkg, oracle_mod, tuning):
    """The product kernels are launched as dependents of the packing kernel (they wait for it on the device, their
    set-up overlapping its end); esmm_tuning_set("NO_DEPENDENT_LAUNCH", 1) launches them the ordinary way.  Tiled and
    strip kernel, same bits."""
    tuning("NO_DEPENDENT_LAUNCH", 1)
    for M, N, K, pa, pb in [(256, 384, 512, 0.5, 0.5), (16, 256, 1024, 0.4, 0.6), (130, 132, 8 * 37, 0.3, 0.7)]:
        A, B = workloads.tile_random(M, N, K, pa, pb, seed=M + N, gran_a=32, gran_b=32)
        check_all_paths(cuda, pkg, oracle_mod, A, B)


def test_gemm_launch_shape_follows_last_call(cuda, pkg, oracle_mod):
    """With PRODUCER_WARPS not pinned, CTA 0 of every launch notes (in a host-mapped word) whether its first tile was
    one of scattered single rows, and the next launch on the device takes the 16-warp form if so.  Alternating
    operands of both kinds, twice each, goes through every transition (12 -> 16 warps, 16 -> 16, 16 -> 12, 12 -> 12);
    every product has the oracle's bits whatever shape it ran in."""
    sparse = workloads.tile_random(512, 512, 2048, 0.2, 0.2, seed=77, gran_a=32, gran_b=32)
    dense = workloads.uniform_pattern(256, 384, 512, 0x0F, seed=78)
    blocks = workloads.block_random(384, 512, 1024, 0.3, 0.4, seed=79)
    forms = []
    for A, B in (dense, sparse, sparse, dense, dense, blocks, sparse, blocks):
        check_all_paths(cuda, pkg, oracle_mod, A, B)
        forms.append(pkg.lib().esmm_last_tiled_kernel_warps())
    # each launch's shape is what the launch before it noted: 16 warps after the scattered operands, 12 after the others
    # (the first one follows whatever ran before this test)
    assert forms[1:] == [12, 16, 16, 12, 12, 12, 16], forms


@pytest.mark.parametrize("form", ["strip", "strip32", "tiled"])
def test_gemm_few_rows(cuda, pkg, oracle_mod, tuning, form):
    """M <= 32 (one pattern block of A) and N >= 128 runs the strip kernel (one CTA per 32 columns), which has a
    16-row variant for M <= 16 (`strip32` forces the 32-row one); the same inputs with that kernel switched off go
    through the tiled kernel.  Same bits as the oracle every way."""
    if form == "tiled":
        tuning("NO_SKINNY", 1)
    if form.endswith("32"):
        tuning("SKINNY_ROWS", 32)
    for M, N, K, pa, pb in [(16, 256, 256, 0.5, 0.5), (32, 1408, 1024, 0.4, 0.6), (1, 128, 64, 1.0, 1.0),
                            (31, 132, 8 * 37, 0.7, 0.3), (8, 512, 4096, 0.2, 0.9), (32, 160, 76, 0.8, 0.8),
                            (24, 256, 2048, 0.0, 0.5), (16, 11008, 4096, 0.4, 0.5), (9, 140, 16384, 0.3, 0.3)]:
        A, B = workloads.tile_random(M, N, K, pa, pb, seed=M + N + K, gran_a=32, gran_b=32)
        check_all_paths(cuda, pkg, oracle_mod, A, B)
    for pat in (0xFF, 0x0F, 0x81):
        A, B = workloads.uniform_pattern(32, 384, 512, pat, seed=pat)
        check_all_paths(cuda, pkg, oracle_mod, A, B)
    A, B = workloads.llm_mlp(16, 1408, 2048, seed=5)
    check_all_paths(cuda, pkg, oracle_mod, A, B)
    A, B = workloads.all_byte_values(M=32, N=256, seed=6)
    check_all_paths(cuda, pkg, oracle_mod, A, B)


@pytest.mark.parametrize("rows", [128, 64])
def test_gemm_block_structured(cuda, pkg, oracle_mod, tuning, rows):
    """Whole 8-deep blocks live or dead (pattern bytes 0x00 / 0xFF), what pruning at the pattern granularity gives:
    the producers fetch whole K blocks, the consumers' masks come in bytes.  Both tilings, same bits as the oracle."""
    tuning("TILE_M", int(rows))
    for M, N, K, pa, pb in [(256, 384, 1024, 0.4, 0.5), (384, 256, 8 * 37, 0.7, 0.3), (200, 132, 512, 0.5, 0.9),
                            (128, 128, 2048, 0.15, 0.15), (256, 256, 512, 1.0, 0.5), (256, 256, 512, 0.5, 1.0)]:
        A, B = workloads.block_random(M, N, K, pa, pb, seed=M + N + K)
        ap = oracle_mod.preprocess_a(A)
        assert set(np.unique(ap)) <= {0, 255}
        check_all_paths(cuda, pkg, oracle_mod, A, B)
    # blocks whose bytes are 0x00 / 0xFF only in some stages: mixed with single live k elsewhere
    A, B = workloads.block_random(256, 256, 1024, 0.5, 0.5, seed=9)
    A[:, 100] = 0.0
    B[300, :] = 0.0
    check_all_paths(cuda, pkg, oracle_mod, A, B)


def test_packing_kernel_variants(cuda, pkg, oracle_mod, tuning):
    """The packing preprocessor has a 32 x 64 task per warp (default) and a 32 x 128 one; both must give the
    oracle's pattern bytes and a packed copy the GEMM turns into the oracle's C (workspace poisoned with NaN
    bit patterns: a dead entry that were read would show)."""
    for variant in ("128", "64"):
        tuning("PACK", int(variant))
        for M, N, K, pa, pb in [(256, 256, 512, 0.5, 0.5), (100, 132, 8 * 37, 0.3, 0.7), (384, 128, 4 * 75, 0.8, 0.4),
                                (16, 256, 256, 0.5, 0.5), (200, 64, 64, 1.0, 1.0)]:
            A, B = workloads.tile_random(M, N, K, pa, pb, seed=M + K, gran_a=32, gran_b=32)
            check_all_paths(cuda, pkg, oracle_mod, A, B)
        A, B = workloads.all_byte_values(seed=31)
        check_all_paths(cuda, pkg, oracle_mod, A, B)


def test_gemm_random_shapes(cuda, pkg, oracle_mod):
    """Seeded random shapes and densities (ragged M, N % 4 == 0, K % 4 == 0, all three kernels and both tilings get
    their share through the launch heuristics): same bits as the oracle everywhere."""
    rng = np.random.default_rng(2024)
    for case in range(40):
        M = int(rng.integers(1, 320))
        N = 4 * int(rng.integers(1, 130))
        K = 4 * int(rng.integers(1, 160))
        pa, pb = float(rng.choice([0.1, 0.3, 0.6, 1.0])), float(rng.choice([0.1, 0.4, 0.8, 1.0]))
        A, B = workloads.tile_random(M, N, K, pa, pb, seed=1000 + case, gran_a=32, gran_b=32)
        if case % 5 == 0:       # a few exact zeros and negative zeros inside live blocks
            A[rng.integers(0, M), :] = 0.0
            B[:, rng.integers(0, N)] = -0.0
        check_all_paths(cuda, pkg, oracle_mod, A, B)


def test_gemm_coarser_and_finer_a_patterns(cuda, pkg, oracle_mod):
    """A pattern granularities of the other joint-sparse kernel ids (64 rows: ids 20/25, 8 rows: id 21)
    give the same C as 32 rows: the extra terms they admit or drop are exact zeros."""
    A, B = workloads.tile_random(256, 256, 512, 0.4, 0.6, seed=13, gran_a=8, gran_b=32)
    d = Dev(cuda, pkg, A, B)
    d.patterns()
    Cref = oracle_mod.gemm_joint(A, B)
    for tile_m in (8, 16, 64, 128):
        ap = cuda.zeros((256 // tile_m, 64), dtype=cuda.uint8, device="cuda")
        pkg.preprocess_a(d.A.data_ptr(), 256, 512, ap.data_ptr(), tile_m=tile_m)
        c = d.C()
        pkg.gemm_ab(256, 256, 512, d.A.data_ptr(), d.B.data_ptr(), c.data_ptr(), ap.data_ptr(), d.bp.data_ptr(),
                    a_tile_m=tile_m)
        pkg.device_status()
        assert oracle_mod.rel_inf_err(c.cpu().numpy(), Cref) <= TOL, tile_m


# ---- golden outputs of the reference's GPU kernels -------------------------------------------------
def test_against_reference_gpu_goldens(cuda, pkg):
    from golden.make_golden import GPU_CASES, make_case
    g = np.load(os.path.join(GOLD, "ref_gpu.npz"))
    for name, M, N, K, gen, args in GPU_CASES:
        A, B = make_case(gen, M, N, K, args)
        d = Dev(cuda, pkg, A, B)
        ap, bp = d.patterns()
        assert np.array_equal(ap, g[name + ".a_pat"]) and np.array_equal(bp, g[name + ".b_pat"]), name
        if name + ".C" in g:
            assert np.array_equal(d.gemm_rowmajor(), g[name + ".C"]), name
            assert np.array_equal(d.sgemm_joint()[0], g[name + ".C"]), name


def test_against_reference_kernels_live(cuda, pkg, oracle_mod):
    """When the compiled reference is present, run its own kernels on the same device buffers."""
    if not oracle_mod.have_ref():
        pytest.skip("oracle/_ref not built")
    R = oracle_mod.ref()
    A, B = workloads.tile_random(512, 512, 1024, 0.35, 0.55, seed=21, gran_a=32, gran_b=32)
    d = Dev(cuda, pkg, A, B)
    ap, bp = d.patterns()
    ra, rb = cuda.zeros_like(d.ap), cuda.zeros_like(d.bp)
    assert R.ref_preprocess_ab_32(d.A.data_ptr(), d.B.data_ptr(), 512, 512, 1024, ra.data_ptr(), rb.data_ptr()) == 0
    assert np.array_equal(ra.cpu().numpy(), ap) and np.array_equal(rb.cpu().numpy(), bp)
    cref = cuda.zeros((512, 512), device="cuda")
    assert R.ref_esmm_v3_launch(512, 512, 1024, d.A.data_ptr(), d.B.data_ptr(), cref.data_ptr(), ra.data_ptr(),
                                rb.data_ptr()) == 0
    cuda.cuda.synchronize()
    assert np.array_equal(d.gemm_rowmajor(), cref.cpu().numpy())
    assert np.array_equal(d.sgemm_joint()[0], cref.cpu().numpy())


def test_skip_stats_against_reference_printout(cuda, pkg, oracle_mod, capfd):
    """The reference's own runner with print_skip_stats = true (include/runners.cuh:843-850) prints the block of
    compute_and_print_skip_stats (:636-706); this library's runner must print the same block, character for
    character, and esmm_skip_stats must return the numbers in it."""
    if not oracle_mod.have_ref():
        pytest.skip("oracle/_ref not built")
    import re
    R = oracle_mod.ref()
    L = pkg.lib()
    M, N, K = 256, 512, 1024
    A, B = workloads.tile_random(M, N, K, 0.25, 0.3, seed=77, gran_a=32, gran_b=32)
    A[64:128] = 0.0                                            # whole CTA rows that skip every K tile
    d = Dev(cuda, pkg, A, B)
    dC = d.C()
    capfd.readouterr()
    assert R.ref_run_esmm_ab_optimized_v3_skip_stats(M, N, K, d.A.data_ptr(), d.B.data_ptr(), dC.data_ptr(), 1) == 1
    cuda.cuda.synchronize()
    C.CDLL(None).fflush(None)
    ref_out = capfd.readouterr().out
    passed, avg = C.c_int(0), C.c_float(0)
    assert L.esmm_run_kernel(29, M, N, K, d.A.data_ptr(), d.B.data_ptr(), dC.data_ptr(), None, None, 1, 0, 1,
                             C.byref(passed), C.byref(avg)) == 0
    C.CDLL(None).fflush(None)                                  # the library prints through C stdio
    our_out = capfd.readouterr().out

    def block(text):
        m = re.search(r"=== Skip Stats: K29 ===\n(.*?\n)\n", text, flags=re.S)
        assert m, text
        return m.group(1)
    assert block(ref_out) == block(our_out)
    nums = [int(x) for x in re.findall(r":\s+(\d+) / (\d+)", block(ref_out))[0:3] for x in x]
    ap, bp = oracle_mod.preprocess_a(A), oracle_mod.preprocess_b(B)
    out = (C.c_longlong * 6)()
    assert L.esmm_skip_stats(ap.ctypes.data, bp.ctypes.data, M // 64, N // 128, K // 8, 2, 4, 8, C.byref(out)) == 0
    assert list(out) == nums
    assert out[0] >= 4 * (K // 8)                              # the zeroed CTA row skips every K tile


# ---- config 1 in full: against the driver's CPU SGEMM -----------------------------------------------
def test_config1_against_cpu_sgemm(cuda, pkg, oracle_mod):
    A, B = workloads.uniform_pattern(1024, 1024, 1024, 0x0F, seed=0)
    d = Dev(cuda, pkg, A, B)
    ap, bp = d.patterns()
    assert set(ap.ravel()) == {0x0F} and set(bp.ravel()) == {0x0F}
    Ccpu = oracle_mod.sgemm_naive(A, B, threads=os.cpu_count() or 1)
    for Cg in (d.gemm_rowmajor(), d.sgemm_joint()[0]):
        assert oracle_mod.rel_inf_err(Cg, Ccpu) <= TOL
        assert oracle_mod.verify_results(Cg, Ccpu, 1e-2)[0] == 0   # the driver's own check


# ---- full benchmark sizes: size-independent properties ------------------------------------------------
@pytest.mark.parametrize("pat", [0xFF, 0x01])
def test_full_size_properties(cuda, pkg, oracle_mod, pat):
    """4096^3 on device-generated inputs: bit-identical to cuBLAS SGEMM on the same (zero-containing)
    matrices would be too strong a claim in general, so check (i) sampled rows against the float64
    oracle, (ii) exact linearity in a power of two, (iii) both kernels agree bit for bit."""
    S = 4096
    t = cuda
    dA = t.empty((S, S), device="cuda")
    dB = t.empty((S, S), device="cuda")
    pkg.fill_normal(dA.data_ptr(), S, S, 0, 1, mode=1, pattern=pat)
    pkg.fill_normal(dB.data_ptr(), S, S, 1, 2, mode=1, pattern=pat)
    ap = t.zeros((S // 32, S // 8), dtype=t.uint8, device="cuda")
    bp = t.zeros_like(ap)
    pkg.preprocess_b(dB.data_ptr(), S, S, bp.data_ptr())
    ws = t.empty(pkg.sgemm_joint_workspace_bytes(S, S), dtype=t.uint8, device="cuda")
    c1 = t.empty((S, S), device="cuda")
    pkg.sgemm_joint(S, S, S, dA.data_ptr(), dB.data_ptr(), c1.data_ptr(), bp.data_ptr(), ws.data_ptr())
    pkg.device_status()
    assert bool((ws[:ap.numel()] == pat).all()) and bool((bp == pat).all())
    rows = [0, 1, 777, 2048, 4095]
    A_rows = dA[rows].cpu().numpy()
    want = oracle_mod.sgemm_f64(A_rows, dB.cpu().numpy())
    assert oracle_mod.rel_inf_err(c1[rows].cpu().numpy(), want) <= TOL
    pkg.preprocess_a(dA.data_ptr(), S, S, ap.data_ptr())
    c2 = t.empty((S, S), device="cuda")
    pkg.gemm_ab(S, S, S, dA.data_ptr(), dB.data_ptr(), c2.data_ptr(), ap.data_ptr(), bp.data_ptr())
    pkg.device_status()
    assert t.equal(c1, c2)
    dA *= 4.0
    pkg.sgemm_joint(S, S, S, dA.data_ptr(), dB.data_ptr(), c2.data_ptr(), bp.data_ptr(), ws.data_ptr())
    pkg.device_status()
    assert t.equal(c2, c1 * 4.0)


# ---- runners, plan, helpers -----------------------------------------------------------------------------
def test_run_kernel_ids(cuda, pkg, oracle_mod, capfd):
    M = N = K = 512
    A, B = workloads.tile_random(M, N, K, 0.5, 0.5, seed=31, gran_a=64, gran_b=32)
    dA, dB = cuda.from_numpy(A).cuda(), cuda.from_numpy(B).cuda()
    dC = cuda.zeros((M, N), device="cuda")
    h_ref = np.zeros((M, N), np.float32)
    L = pkg.lib()
    passed, avg = C.c_int(0), C.c_float(0)
    # id 15 fills the reference result, like the driver does with cuBLAS
    assert L.esmm_run_kernel(15, M, N, K, dA.data_ptr(), dB.data_ptr(), dC.data_ptr(), h_ref.ctypes.data, None, 2, 0,
                             0, C.byref(passed), C.byref(avg)) == 0
    assert oracle_mod.rel_inf_err(h_ref, oracle_mod.sgemm_f64(A, B)) <= TOL
    h_c = np.zeros((M, N), np.float32)
    for kid in (29, 20, 21, 25, 26, 27, 28, 30):
        st = L.esmm_run_kernel(kid, M, N, K, dA.data_ptr(), dB.data_ptr(), dC.data_ptr(), h_c.ctypes.data,
                               h_ref.ctypes.data, 2, 1, int(kid == 29), C.byref(passed), C.byref(avg))
        assert st == 0 and passed.value == 1 and avg.value > 0, kid
        assert oracle_mod.rel_inf_err(h_c, h_ref) <= TOL
    out = capfd.readouterr().out
    assert out.count("Kernel time:") == 9 and "=== Skip Stats: K29 ===" in out
    # single-operand ids: 16 (A patterns, B all live) and 17 (B patterns) give the joint kernel's bits
    h_29 = h_c.copy()
    for kid in (16, 17):
        st = L.esmm_run_kernel(kid, M, N, K, dA.data_ptr(), dB.data_ptr(), dC.data_ptr(), h_c.ctypes.data,
                               h_ref.ctypes.data, 1, 1, 0, C.byref(passed), C.byref(avg))
        assert st == 0 and passed.value == 1, kid
        assert np.array_equal(h_c, h_29), kid
    capfd.readouterr()
    h_bad = h_ref + 1.0
    st = L.esmm_run_kernel(29, M, N, K, dA.data_ptr(), dB.data_ptr(), dC.data_ptr(), h_c.ctypes.data,
                           h_bad.ctypes.data, 1, 1, 0, C.byref(passed), C.byref(avg))
    assert st == pkg.ERR_VERIFY and passed.value == 0
    assert "Verification failed" in capfd.readouterr().out


def test_run_kernel_prefix_pattern(cuda, pkg, oracle_mod, capfd):
    """Id 14 multiplies the first popcount(pattern) k of every 8-slice whatever the data holds
    (include/runners.cuh:47-66): on a dense A the result is the product with A's other columns dropped."""
    M, N, K = 256, 384, 512
    rng = np.random.default_rng(77)
    A = rng.standard_normal((M, K), dtype=np.float32)
    B = rng.standard_normal((K, N), dtype=np.float32)
    dA, dB = cuda.from_numpy(A).cuda(), cuda.from_numpy(B).cuda()
    dC = cuda.zeros((M, N), device="cuda")
    L = pkg.lib()
    passed, avg = C.c_int(0), C.c_float(0)
    for pat, live in ((b"11110000", 4), (b"10000001", 2), (b"11111111", 8), (b"00000001", 1), (b"11101110", 6)):
        st = L.esmm_run_kernel_pattern(14, M, N, K, dA.data_ptr(), dB.data_ptr(), dC.data_ptr(), None, None, 1, 0, 0,
                                       None, pat, C.byref(passed), C.byref(avg))
        assert st == 0 and passed.value == 1
        Am = A.copy()
        Am[:, (np.arange(K) % 8) >= live] = 0.0
        a_pat = np.full((M // 32, K // 8), (1 << live) - 1, np.uint8)
        b_pat = np.full((N // 32, K // 8), 0xFF, np.uint8)
        assert np.array_equal(dC.cpu().numpy(), oracle_mod.gemm_joint(A, B, a_pat, b_pat)), pat
        assert oracle_mod.rel_inf_err(dC.cpu().numpy(), oracle_mod.sgemm_f64(Am, B)) <= TOL
    # a count without an unrolled kernel: nothing runs, C stays zero
    st = L.esmm_run_kernel_pattern(14, M, N, K, dA.data_ptr(), dB.data_ptr(), dC.data_ptr(), None, None, 1, 0, 0,
                                   None, b"11100000", C.byref(passed), C.byref(avg))
    assert st == 0 and float(dC.abs().max()) == 0.0
    assert L.esmm_run_kernel_pattern(14, M, N, K, dA.data_ptr(), dB.data_ptr(), dC.data_ptr(), None, None, 1, 0, 0,
                                     None, b"111", C.byref(passed), C.byref(avg)) == pkg.ERR_SHAPE
    capfd.readouterr()


def test_plan_host_buffers(cuda, pkg, oracle_mod):
    M, N, K = 640, 384, 512
    A, B = workloads.tile_random(M, N, K, 0.4, 0.6, seed=41, gran_a=32, gran_b=32)
    hA = cuda.from_numpy(A).pin_memory()
    hC = cuda.empty((M, N)).pin_memory()
    Cref = oracle_mod.gemm_joint(A, B)
    for chunks in (1, 3, 64):
        plan = C.c_void_p()
        pkg.check(pkg.lib().esmm_plan_create(M, N, K, B.ctypes.data, chunks, C.byref(plan)), "plan_create")
        hC.fill_(float("nan"))
        pkg.check(pkg.lib().esmm_plan_run(plan, hA.data_ptr(), hC.data_ptr()), "plan_run")
        assert np.array_equal(hC.numpy(), Cref), chunks
        pkg.check(pkg.lib().esmm_plan_run(plan, hA.data_ptr(), hC.data_ptr()), "plan_run twice")
        assert np.array_equal(hC.numpy(), Cref), chunks
        pkg.lib().esmm_plan_destroy(plan)
    # several submissions in flight on one plan (different inputs, own result buffers) and on a second plan
    L = pkg.lib()
    A2 = A[::-1].copy()
    Cref2 = oracle_mod.gemm_joint(A2, B)
    hA2, hC2, hC3 = cuda.from_numpy(A2).pin_memory(), cuda.empty((M, N)).pin_memory(), cuda.empty((M, N)).pin_memory()
    p1, p2 = C.c_void_p(), C.c_void_p()
    pkg.check(L.esmm_plan_create(M, N, K, B.ctypes.data, 3, C.byref(p1)), "plan_create")
    pkg.check(L.esmm_plan_create(M, N, K, B.ctypes.data, 2, C.byref(p2)), "plan_create")
    for rep in range(3):
        for h in (hC, hC2, hC3):
            h.fill_(float("nan"))
        pkg.check(L.esmm_plan_submit(p1, hA.data_ptr(), hC.data_ptr()), "submit")
        pkg.check(L.esmm_plan_submit(p1, hA2.data_ptr(), hC2.data_ptr()), "submit")
        pkg.check(L.esmm_plan_submit(p2, hA2.data_ptr(), hC3.data_ptr()), "submit")
        pkg.check(L.esmm_plan_wait(p1), "wait")
        pkg.check(L.esmm_plan_wait(p2), "wait")
        assert np.array_equal(hC.numpy(), Cref) and np.array_equal(hC2.numpy(), Cref2) and np.array_equal(hC3.numpy(), Cref2)
    L.esmm_plan_destroy(p1)
    L.esmm_plan_destroy(p2)
    assert L.esmm_plan_submit(None, hA.data_ptr(), hC.data_ptr()) == pkg.ERR_NULL and L.esmm_plan_wait(None) == pkg.ERR_NULL


def test_cublas_and_generators(cuda, pkg, oracle_mod):
    S = 512
    dA = cuda.empty((S, S), device="cuda")
    dB = cuda.empty((S, S), device="cuda")
    pkg.fill_normal(dA.data_ptr(), S, S, 0, 7, mode=2, p_live=0.3, gran=64, seed2=1)
    pkg.fill_normal(dB.data_ptr(), S, S, 1, 8, mode=2, p_live=0.7, gran=64, seed2=2)
    A, B = dA.cpu().numpy(), dB.cpu().numpy()
    ap, bp = oracle_mod.preprocess_a(A), oracle_mod.preprocess_b(B)
    assert np.array_equal(ap[0::2], ap[1::2]) and np.array_equal(bp[0::2], bp[1::2])
    da = np.unpackbits(ap, bitorder="little").mean()
    db = np.unpackbits(bp, bitorder="little").mean()
    assert da == pytest.approx(0.3, abs=0.03) and db == pytest.approx(0.7, abs=0.03)
    live = A[A != 0]
    assert abs(live.mean()) < 0.02 and live.std() == pytest.approx(1.0, abs=0.02)
    dC = cuda.empty((S, S), device="cuda")
    pkg.cublas_sgemm(S, S, S, dA.data_ptr(), dB.data_ptr(), dC.data_ptr())
    cuda.cuda.synchronize()
    assert oracle_mod.rel_inf_err(dC.cpu().numpy(), oracle_mod.sgemm_f64(A, B)) <= TOL
    # same seed -> same matrix; relu and mean/std parameters
    dA2 = cuda.empty((S, S), device="cuda")
    pkg.fill_normal(dA2.data_ptr(), S, S, 0, 7, mode=2, p_live=0.3, gran=64, seed2=1)
    assert cuda.equal(dA, dA2)
    pkg.fill_normal(dA2.data_ptr(), S, S, 0, 9, mean=0.0, std=0.02, relu=True)
    x = dA2.cpu().numpy()
    assert x.min() == 0.0 and x.max() < 0.2 and (x == 0).mean() == pytest.approx(0.5, abs=0.02)


def test_interleave_shards(cuda, pkg):
    M, N, G = 96, 256, 4
    full = np.random.default_rng(3).standard_normal((M, N), dtype=np.float32)
    shards = np.stack([full[:, g * (N // G):(g + 1) * (N // G)] for g in range(G)])
    dS = cuda.from_numpy(np.ascontiguousarray(shards)).cuda()
    dC = cuda.zeros((M, N), device="cuda")
    pkg.check(pkg.lib().esmm_interleave_shards(dS.data_ptr(), dC.data_ptr(), M, N, G, 0), "interleave")
    cuda.cuda.synchronize()
    assert np.array_equal(dC.cpu().numpy(), full)


def test_ffma_peak_is_plausible(pkg, cuda):
    tf, sms = pkg.ffma_peak_tflops()
    assert sms >= 100 and 30.0 < tf < 90.0


def test_smoke_entry(cuda):
    import __graft_entry__ as g
    g.smoke()


def test_bounded_wait_reports_timeout_and_context_survives(cuda, pkg, oracle_mod):
    """A device-side wait that nothing satisfies gives up after its budget, the kernel returns and
    the host reads ESMM_ERR_TIMEOUT; the next call works and the status is clean again."""
    L = pkg.lib()
    assert L.esmm_device_status(None) == 0
    assert L.esmm_selftest_bounded_wait(2000, None) == 0          # 2 ms budget
    assert L.esmm_device_status(None) == pkg.ERR_TIMEOUT
    assert L.esmm_device_status(None) == 0                        # reading clears it
    assert L.esmm_selftest_bounded_wait(0, None) == pkg.ERR_SHAPE
    assert L.esmm_selftest_bounded_wait(2_000_000, None) == pkg.ERR_SHAPE
    A, B = workloads.uniform_pattern(128, 128, 64, 0x0F, seed=3)
    check_all_paths(cuda, pkg, oracle_mod, A, B)


def test_gemm_mask_builder_paths_agree(cuda, pkg, oracle_mod, tuning):
    """The tile's row list is built from 16-byte pattern loads (long K), 4-byte loads (shorter K) or byte
    by byte (pattern rows that are not a multiple of 4 bytes); all must give the same C."""
    A, B = workloads.tile_random(256, 384, 8192 + 128, 0.3, 0.5, seed=17, gran_a=32, gran_b=32)  # 1040 K blocks
    for mode in ("0", "4", "16"):
        tuning("VEC_PATTERNS", int(mode))
        check_all_paths(cuda, pkg, oracle_mod, A, B)
    tuning.reset()
    A, B = workloads.tile_random(256, 256, 8 * 37, 0.5, 0.5, seed=18, gran_a=32, gran_b=32)      # 37 K blocks: bytes
    check_all_paths(cuda, pkg, oracle_mod, A, B)


def test_multi_launcher_two_ranks_on_one_gpu(cuda, pkg, oracle_mod):
    """The C++ sharded launcher (esmm_multi_*) with both ranks placed on device 0: column shards computed by two host
    threads on two streams must reproduce the unsharded result bit for bit (the shards' kernels are independent -
    none waits on another).  The NCCL gather refuses a device named twice; the shards come back by download."""
    L = pkg.lib()
    M, N, K = 256, 512, 512
    A, B = workloads.tile_random(M, N, K, 0.5, 0.5, seed=91, gran_a=32, gran_b=32)
    want = Dev(cuda, pkg, A, B)
    want.patterns()
    Cwant, _ = want.sgemm_joint()
    h = C.c_void_p()
    devs = (C.c_int * 2)(0, 0)
    pkg.check(L.esmm_multi_create(M, N, K, 2, devs, C.byref(h)), "esmm_multi_create")
    try:
        assert L.esmm_multi_num_gpus(h) == 2
        assert L.esmm_multi_run(h, 1, None, None) == pkg.ERR_NULL                 # nothing uploaded yet
        pkg.check(L.esmm_multi_upload(h, A.ctypes.data, B.ctypes.data), "esmm_multi_upload")
        ms_max, ms = C.c_float(0), (C.c_float * 2)()
        pkg.check(L.esmm_multi_run(h, 3, C.byref(ms_max), ms), "esmm_multi_run")
        assert ms_max.value > 0 and ms_max.value == max(ms[0], ms[1])
        got = np.full((M, N), np.nan, np.float32)
        pkg.check(L.esmm_multi_download(h, got.ctypes.data), "esmm_multi_download")
        assert np.array_equal(got, Cwant) and np.array_equal(got, oracle_mod.gemm_joint(A, B))
        assert L.esmm_multi_gather(h, None, None) == pkg.ERR_UNSUPPORTED            # one rank per device only
    finally:
        L.esmm_multi_destroy(h)
    bad = (C.c_int * 2)(0, 99)
    assert L.esmm_multi_create(M, N, K, 2, bad, C.byref(h)) == pkg.ERR_UNSUPPORTED
