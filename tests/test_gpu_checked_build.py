"""The sanitizer substitute: (1) the bounds-checked build of the library (libesmm_b200_checked.so, -DESMM_CHECKED) runs
the small parity shapes - ragged ones included - and reports no out-of-range index; (2) with BOTH builds every device
buffer a call may write (C, the workspace, the pattern arrays) sits between canary margins that must be intact
afterwards, and every buffer it may only read is followed by a poisoned margin (NaN bit patterns) that would show in C if
it were read.  The failure report itself is exercised by a kernel that reports a failed check without making any access:
nothing here faults a GPU."""
import numpy as np
import pytest

import workloads

pytestmark = pytest.mark.gpu
MARGIN = 4096          # bytes of canary on each side of a writable buffer
CANARY = 0xA5

SHAPES = [  # (M, N, K, pA, pB): small, odd and ragged shapes of the parity tests
    (64, 128, 64, 0.5, 0.5), (128, 128, 8, 1.0, 1.0), (100, 132, 8 * 37, 0.3, 0.7), (257, 260, 1000, 0.4, 0.4),
    (16, 256, 256, 0.5, 0.5), (33, 64, 72, 0.6, 0.6), (384, 128, 4 * 75, 0.8, 0.4), (200, 64, 64, 1.0, 1.0),
    (512, 384, 1024, 0.2, 0.2), (64, 512, 8 * 1025, 0.1, 0.5),
]


class Guarded:
    """A device buffer of `nbytes` with a canary margin before and after it."""

    def __init__(self, t, nbytes, fill=0xEE):
        self.t, self.n = t, nbytes
        self.pad = (MARGIN + 255) & ~255
        self.raw = t.full((self.pad + ((nbytes + 255) & ~255) + self.pad,), CANARY, dtype=t.uint8, device="cuda")
        self.raw[self.pad:self.pad + nbytes] = fill

    @property
    def ptr(self):
        return self.raw.data_ptr() + self.pad

    def view(self, dtype, shape):
        return self.raw[self.pad:self.pad + self.n].view(dtype).reshape(shape)

    def intact(self):
        head = self.raw[:self.pad]
        tail = self.raw[self.pad + self.n:]
        return bool((head == CANARY).all()) and bool((tail == CANARY).all())


def read_only(t, arr):
    """Input matrix followed by a poisoned margin (NaN bit patterns): reading past the end would poison C."""
    flat = np.ascontiguousarray(arr).view(np.uint8).ravel()
    buf = t.full((flat.size + MARGIN,), 0xFF, dtype=t.uint8, device="cuda")
    buf[:flat.size] = t.from_numpy(flat.copy()).cuda()
    return buf


@pytest.fixture(scope="module")
def libs(pkg):
    return {"product": pkg.lib(), "checked": pkg.load_library(pkg.CHECKED_LIB_PATH)}


def test_checked_build_reports_without_faulting(cuda, pkg, libs, request):
    """esmm_selftest_bounds_report makes no access at all: it only files the report.  The checked build answers
    ESMM_ERR_BOUNDS with the site number, the product build (checks compiled out) ESMM_OK; both contexts stay usable."""
    if request.config.getoption("--checked-lib"):
        pytest.skip("the product library is replaced by the checked build in this run")
    assert libs["checked"].esmm_checked_build() == 1 and libs["product"].esmm_checked_build() == 0
    for name, L in libs.items():
        assert L.esmm_device_status(None) == 0
        assert L.esmm_selftest_bounds_report(None) == 0
        st = L.esmm_device_status(None)
        if name == "checked":
            assert st == pkg.ERR_BOUNDS and b"site 99" in L.esmm_last_cuda_error()
        else:
            assert st == 0
        assert L.esmm_device_status(None) == 0          # the word is cleared by the read


@pytest.mark.parametrize("which", ["checked", "product"])
@pytest.mark.parametrize("M,N,K,pA,pB", SHAPES)
def test_guarded_buffers_and_bounds_checks(cuda, pkg, libs, oracle_mod, which, M, N, K, pA, pB):
    t, L = cuda, libs[which]
    A, B = workloads.tile_random(M, N, K, pA, pB, seed=M + N + K, gran_a=32, gran_b=32)
    dA, dB = read_only(t, A), read_only(t, B)
    nkb = -(-K // 8)
    ap = Guarded(t, -(-M // 32) * nkb)
    bp = Guarded(t, -(-N // 32) * nkb)
    c1 = Guarded(t, M * N * 4, fill=0xFF)
    c2 = Guarded(t, M * N * 4, fill=0xFF)
    ws = Guarded(t, int(L.esmm_sgemm_joint_workspace_bytes(M, K)), fill=0xFF)
    # pattern preprocessors, the row-major kernel, then the per-call path (packing preprocess + packed / strip kernel)
    assert L.esmm_preprocess_a(dA.data_ptr(), M, K, 32, ap.ptr, None) == 0
    assert L.esmm_preprocess_b(dB.data_ptr(), K, N, bp.ptr, None) == 0
    assert L.esmm_gemm_ab(M, N, K, dA.data_ptr(), dB.data_ptr(), c1.ptr, ap.ptr, bp.ptr, 32, None) == 0
    assert L.esmm_sgemm_joint(M, N, K, dA.data_ptr(), dB.data_ptr(), c2.ptr, bp.ptr, ws.ptr, None) == 0
    st = L.esmm_device_status(None)
    assert st == 0, (st, L.esmm_last_cuda_error())
    for name, g in (("A patterns", ap), ("B patterns", bp), ("C (row-major kernel)", c1), ("C (per-call path)", c2),
                    ("workspace", ws)):
        assert g.intact(), f"{which} build wrote outside {name}"
    oap, obp = oracle_mod.preprocess_a(A), oracle_mod.preprocess_b(B)
    assert np.array_equal(ap.view(t.uint8, oap.shape).cpu().numpy(), oap)
    assert np.array_equal(bp.view(t.uint8, obp.shape).cpu().numpy(), obp)
    want = oracle_mod.gemm_joint(A, B, oap, obp)
    for g in (c1, c2):
        got = g.view(t.float32, (M, N)).cpu().numpy()
        assert not np.isnan(got).any() and np.array_equal(got, want)


@pytest.mark.parametrize("which", ["checked", "product"])
@pytest.mark.parametrize("hook,value", [(b"PRODUCER_WARPS", 0), (b"PRODUCER_WARPS", 7)])
def test_guarded_buffers_sixteen_warp_form(cuda, pkg, libs, oracle_mod, which, hook, value):
    """The 16-warp launch shape of the tiled kernel, pinned (its per-CTA choice of copying producers, and all 7 copying),
    on scattered, ragged and block-dense shapes: same guards, no bounds report, the oracle's bits."""
    t, L = cuda, libs[which]
    assert L.esmm_tuning_set(hook, value) == 0
    try:
        for M, N, K, pA, pB in [(512, 384, 1024, 0.2, 0.2), (257, 260, 1000, 0.4, 0.4), (100, 132, 8 * 37, 0.3, 0.7),
                                (200, 64, 64, 1.0, 1.0), (64, 512, 8 * 1025, 0.1, 0.5)]:
            A, B = workloads.tile_random(M, N, K, pA, pB, seed=M + N + K, gran_a=32, gran_b=32)
            dA, dB = read_only(t, A), read_only(t, B)
            bp = Guarded(t, -(-N // 32) * -(-K // 8))
            c = Guarded(t, M * N * 4, fill=0xFF)
            ws = Guarded(t, int(L.esmm_sgemm_joint_workspace_bytes(M, K)), fill=0xFF)
            assert L.esmm_preprocess_b(dB.data_ptr(), K, N, bp.ptr, None) == 0
            assert L.esmm_sgemm_joint(M, N, K, dA.data_ptr(), dB.data_ptr(), c.ptr, bp.ptr, ws.ptr, None) == 0
            st = L.esmm_device_status(None)
            assert st == 0, (st, L.esmm_last_cuda_error())
            assert bp.intact() and c.intact() and ws.intact(), (M, N, K)
            got = c.view(t.float32, (M, N)).cpu().numpy()
            assert not np.isnan(got).any() and np.array_equal(got, oracle_mod.gemm_joint(A, B)), (M, N, K)
    finally:
        L.esmm_tuning_reset()


@pytest.mark.parametrize("which", ["checked", "product"])
def test_guarded_buffers_other_granularities_and_tf32(cuda, pkg, libs, oracle_mod, which):
    """The A pattern kernel at 8 / 64-row granularity and the optional tensor-core variant, same guards."""
    import ctypes as C
    t, L = cuda, libs[which]
    M, N, K = 192, 256, 512
    A, B = workloads.tile_random(M, N, K, 0.4, 0.5, seed=3, gran_a=64, gran_b=32)
    dA, dB = read_only(t, A), read_only(t, B)
    for tile_m in (8, 64):
        g = Guarded(t, -(-M // tile_m) * (K // 8))
        assert L.esmm_preprocess_a(dA.data_ptr(), M, K, tile_m, g.ptr, None) == 0
        assert L.esmm_device_status(None) == 0 and g.intact()
        want = oracle_mod.preprocess_a(A, tile_m)
        assert np.array_equal(g.view(t.uint8, want.shape).cpu().numpy(), want)
    h = C.c_void_p()
    assert L.esmm_tf32x3_b_create(dB.data_ptr(), K, N, 1, C.byref(h)) == 0
    try:
        ws = Guarded(t, int(L.esmm_tf32x3_workspace_bytes(M, K)), fill=0xFF)
        c = Guarded(t, M * N * 4, fill=0xFF)
        assert L.esmm_sgemm_joint_tf32x3(M, dA.data_ptr(), h, c.ptr, ws.ptr, None) == 0
        assert L.esmm_device_status(None) == 0 and ws.intact() and c.intact()
        got = c.view(t.float32, (M, N)).cpu().numpy()
        assert oracle_mod.rel_inf_err(got, oracle_mod.gemm_joint(A, B)) <= 1e-5
    finally:
        L.esmm_tf32x3_b_destroy(h)
