"""ctypes front-end of the CPU oracle (oracle/esmm_oracle.c) and, when it has been
built, of the unmodified reference compiled into oracle/_ref/libesmm_ref.so.

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the
benchmark's CPU-baseline leg.  The product package never imports this module.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from concurrent.futures import ThreadPoolExecutor

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")
_REF_PATH = os.path.join(_HERE, "_ref", "libesmm_ref.so")
SWAPPED_EXE = os.path.join(_HERE, "_ref", "exec_swapped")   # the reference driver.cu built against this repository

_f32p = np.ctypeslib.ndpointer(dtype=np.float32, flags="C_CONTIGUOUS")
_f64p = np.ctypeslib.ndpointer(dtype=np.float64, flags="C_CONTIGUOUS")
_u8p = np.ctypeslib.ndpointer(dtype=np.uint8, flags="C_CONTIGUOUS")
_i64p = np.ctypeslib.ndpointer(dtype=np.int64, flags="C_CONTIGUOUS")


def ref_root() -> str:
    """Where the reference tree is looked for: $ESMM_REF_ROOT, else a directory named `reference`
    beside the repository."""
    return os.environ.get("ESMM_REF_ROOT") or os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")


def have_ref_tree() -> bool:
    return os.path.exists(os.path.join(ref_root(), "include", "runners.cuh"))


def build(force: bool = False) -> None:
    """Compile liboracle.so (and oracle/_ref when the reference tree is present)."""
    src = os.path.join(_HERE, "esmm_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "oracle"])
    shim = os.path.join(_HERE, "ref_shim.cu")
    if have_ref_tree():
        if force or not os.path.exists(_REF_PATH) or os.path.getmtime(_REF_PATH) < os.path.getmtime(shim):
            subprocess.check_call(["make", "-C", _HERE, "ref", f"REF_ROOT={ref_root()}"])
        # the reference's own driver against this repository's headers and library (run by a GPU test)
        lib = os.path.join(os.path.dirname(_HERE), "esmm-research_b200", "libesmm_b200.so")
        inc = [os.path.join(os.path.dirname(_HERE), "include", h) for h in ("utils.cuh", "runners.cuh", "esmm.h")]
        if os.path.exists(lib):
            newest = max(os.path.getmtime(f) for f in inc + [lib])
            if force or not os.path.exists(SWAPPED_EXE) or os.path.getmtime(SWAPPED_EXE) < newest:
                subprocess.check_call(["make", "-C", _HERE, "swapped", f"REF_ROOT={ref_root()}"])


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        L = C.CDLL(_LIB_PATH)
        L.oracle_preprocess_a.argtypes = [_f32p, C.c_int, C.c_int, C.c_int, _u8p]
        L.oracle_preprocess_b.argtypes = [_f32p, C.c_int, C.c_int, C.c_int, _u8p]
        L.oracle_gemm_joint.argtypes = [C.c_int, C.c_int, C.c_int, _f32p, _f32p, _f32p, _u8p, _u8p,
                                        C.c_int, C.c_int]
        L.oracle_sgemm_naive_rows.argtypes = [_f32p, _f32p, _f32p, C.c_int, C.c_int, C.c_int,
                                              C.c_int, C.c_int]
        L.oracle_sgemm_f64_rows.argtypes = [_f32p, _f32p, _f64p, C.c_int, C.c_int, C.c_int,
                                            C.c_int, C.c_int]
        L.oracle_verify_results.argtypes = [_f32p, _f32p, C.c_long, C.c_float,
                                            C.POINTER(C.c_float), C.POINTER(C.c_long)]
        L.oracle_verify_results.restype = C.c_long
        L.oracle_skip_stats.argtypes = [_u8p, _u8p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                        C.c_int, _i64p]
        L.oracle_pattern_from_string.argtypes = [C.c_char_p]
        L.oracle_pattern_from_string.restype = C.c_int
        L.oracle_pattern_lut.argtypes = [C.c_uint8, C.POINTER(C.c_uint8), C.POINTER(C.c_uint8 * 8)]
        L.oracle_executed_macs.argtypes = [_u8p, _u8p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int]
        L.oracle_executed_macs.restype = C.c_longlong
        _lib = L
    return _lib


def _c(a, dt=np.float32):
    return np.ascontiguousarray(a, dtype=dt)


def preprocess_a(A: np.ndarray, tile_m: int = 32) -> np.ndarray:
    A = _c(A)
    M, K = A.shape
    out = np.zeros((-(-M // tile_m), -(-K // 8)), np.uint8)
    lib().oracle_preprocess_a(A, M, K, tile_m, out)
    return out


def preprocess_b(B: np.ndarray, wn: int = 32) -> np.ndarray:
    B = _c(B)
    K, N = B.shape
    out = np.zeros((-(-N // wn), -(-K // 8)), np.uint8)
    lib().oracle_preprocess_b(B, K, N, wn, out)
    return out


def gemm_joint(A, B, a_pat=None, b_pat=None, tile_m: int = 32, wn: int = 32) -> np.ndarray:
    A, B = _c(A), _c(B)
    M, K = A.shape
    K2, N = B.shape
    assert K == K2
    a_pat = preprocess_a(A, tile_m) if a_pat is None else _c(a_pat, np.uint8)
    b_pat = preprocess_b(B, wn) if b_pat is None else _c(b_pat, np.uint8)
    Cm = np.empty((M, N), np.float32)
    lib().oracle_gemm_joint(M, N, K, A, B, Cm, a_pat, b_pat, tile_m, wn)
    return Cm


def sgemm_naive(A, B, rows=None, threads: int = 1) -> np.ndarray:
    """The driver's CPU SGEMM loop nest; `rows=(r0, r1)` computes a slab, `threads`
    splits the slab's rows across host threads (results do not depend on it)."""
    A, B = _c(A), _c(B)
    M, K = A.shape
    N = B.shape[1]
    r0, r1 = (0, M) if rows is None else rows
    Cm = np.zeros((M, N), np.float32)
    L = lib()
    if threads <= 1:
        L.oracle_sgemm_naive_rows(A, B, Cm, M, N, K, r0, r1)
    else:
        cuts = np.linspace(r0, r1, threads + 1).astype(int)
        with ThreadPoolExecutor(threads) as ex:
            list(ex.map(lambda ab: L.oracle_sgemm_naive_rows(A, B, Cm, M, N, K, int(ab[0]), int(ab[1])),
                        zip(cuts[:-1], cuts[1:])))
    return Cm[r0:r1] if rows is not None else Cm


def sgemm_f64(A, B, rows=None) -> np.ndarray:
    A, B = _c(A), _c(B)
    M, K = A.shape
    N = B.shape[1]
    r0, r1 = (0, M) if rows is None else rows
    out = np.empty((r1 - r0, N), np.float64)
    lib().oracle_sgemm_f64_rows(A, B, out, M, N, K, r0, r1)
    return out


def verify_results(gpu, ref, tol: float = 1e-2):
    gpu, ref = _c(gpu).ravel(), _c(ref).ravel()
    md, fi = C.c_float(0), C.c_long(-1)
    bad = lib().oracle_verify_results(gpu, ref, gpu.size, tol, C.byref(md), C.byref(fi))
    return int(bad), float(md.value), int(fi.value)


def skip_stats(a_pat, b_pat, warps_m: int, warps_n: int, bk: int = 8) -> dict:
    a_pat, b_pat = _c(a_pat, np.uint8), _c(b_pat, np.uint8)
    nKB = a_pat.shape[1]
    out = np.zeros(6, np.int64)
    lib().oracle_skip_stats(a_pat, b_pat, a_pat.shape[0] // warps_m, b_pat.shape[0] // warps_n, nKB,
                            warps_m, warps_n, bk, out)
    keys = ["block_skips", "total_k", "warp_skips", "total_warp_k", "dot_skips", "total_dot"]
    return dict(zip(keys, (int(x) for x in out)))


def pattern_from_string(s: str) -> int:
    return lib().oracle_pattern_from_string(s.encode())


def pattern_lut(p: int):
    cnt = C.c_uint8(0)
    off = (C.c_uint8 * 8)()
    lib().oracle_pattern_lut(p, C.byref(cnt), C.byref(off))
    return int(cnt.value), list(off)


def executed_macs(a_pat, b_pat, tile_m: int = 32, wn: int = 32) -> int:
    a_pat, b_pat = _c(a_pat, np.uint8), _c(b_pat, np.uint8)
    return int(lib().oracle_executed_macs(a_pat, b_pat, a_pat.shape[0], b_pat.shape[0],
                                          a_pat.shape[1], tile_m, wn))


def rel_inf_err(Cm, Cref) -> float:
    """max|C - C_ref| / max|C_ref|: the tolerance metric of the parity tests."""
    Cref = np.asarray(Cref, np.float64)
    den = float(np.max(np.abs(Cref)))
    num = float(np.max(np.abs(np.asarray(Cm, np.float64) - Cref)))
    return num / den if den > 0 else num


# ---------------------------------------------------------------------------
# The unmodified reference (oracle/_ref), when built.
# ---------------------------------------------------------------------------
_ref = None


def have_ref() -> bool:
    return os.path.exists(_REF_PATH)


def ref() -> C.CDLL:
    """oracle/_ref/libesmm_ref.so: host functions work without a GPU; the ref_*
    GPU entry points take raw device pointers (integers)."""
    global _ref
    if _ref is None:
        R = C.CDLL(_REF_PATH)
        R.ref_matrixMultiplyCPU.argtypes = [_f32p, _f32p, _f32p, C.c_int, C.c_int, C.c_int]
        R.ref_matrixMultiplyCPU_rows.argtypes = [_f32p, _f32p, _f32p, C.c_int, C.c_int, C.c_int,
                                                 C.c_int, C.c_int]
        R.ref_verifyResults.argtypes = [_f32p, _f32p, C.c_int, C.c_float]
        R.ref_randomize_A_blocklevel_8_32.argtypes = [_f32p, C.c_int, C.c_int, C.c_float, C.c_uint]
        R.ref_randomize_B_blocklevel_8_32.argtypes = [_f32p, C.c_int, C.c_int, C.c_float, C.c_uint]
        R.ref_randomize_A_8_8.argtypes = [_f32p, C.c_int, C.c_int, C.c_float, C.c_uint]
        R.ref_randomize_with_pattern.argtypes = [_f32p, C.c_int, C.c_int, C.c_char_p]
        R.ref_randomize_unstructured.argtypes = [_f32p, C.c_int, C.c_int, C.c_float, C.c_uint]
        R.ref_srand.argtypes = [C.c_uint]
        R.ref_parse_kernel_selection.argtypes = [C.c_char_p, C.POINTER(C.c_int), C.c_int]
        R.ref_get_kernel_name.argtypes = [C.c_int]
        R.ref_get_kernel_name.restype = C.c_char_p
        vp = C.c_void_p
        R.ref_preprocess_ab_32.argtypes = [vp, vp, C.c_int, C.c_int, C.c_int, vp, vp]
        R.ref_esmm_v3_launch.argtypes = [C.c_int, C.c_int, C.c_int, vp, vp, vp, vp, vp]
        R.ref_run_esmm_ab_optimized_v3_no_check.argtypes = [C.c_int, C.c_int, C.c_int, vp, vp, vp, C.c_int]
        fp = C.POINTER(C.c_float)
        R.ref_time_kernels_v3.argtypes = [C.c_int, C.c_int, C.c_int, vp, vp, vp, vp, vp, C.c_int, C.c_int, fp, fp, fp]
        R.ref_run_esmm_ab_optimized_v3_skip_stats.argtypes = [C.c_int, C.c_int, C.c_int, vp, vp, vp, C.c_int]
        _ref = R
    return _ref


def ref_time_kernels(M, N, K, d_A, d_B, d_C, d_a_pat, d_b_pat, warmup=2, runs=5):
    """(ms preprocess A, ms preprocess B, ms kernel id 29) of the reference's own kernels on device buffers
    (raw pointers), CUDA-event averages; raises if the shape is outside the reference kernel's limits."""
    a, b, g = C.c_float(0), C.c_float(0), C.c_float(0)
    e = ref().ref_time_kernels_v3(M, N, K, d_A, d_B, d_C, d_a_pat, d_b_pat, warmup, runs,
                                  C.byref(a), C.byref(b), C.byref(g))
    if e != 0:
        raise RuntimeError(f"reference kernels failed or shape unsupported: cudaError {e}")
    return float(a.value), float(b.value), float(g.value)


def ref_sgemm_cpu(A, B, rows=None, threads: int = 1) -> np.ndarray:
    """matrixMultiplyCPU of the reference itself, optionally on a row slab / threaded."""
    A, B = _c(A), _c(B)
    M, K = A.shape
    N = B.shape[1]
    r0, r1 = (0, M) if rows is None else rows
    Cm = np.zeros((M, N), np.float32)
    R = ref()
    cuts = np.linspace(r0, r1, max(1, threads) + 1).astype(int)
    with ThreadPoolExecutor(max(1, threads)) as ex:
        list(ex.map(lambda ab: R.ref_matrixMultiplyCPU_rows(A, B, Cm, M, N, K, int(ab[0]), int(ab[1])),
                    zip(cuts[:-1], cuts[1:])))
    return Cm[r0:r1] if rows is not None else Cm
