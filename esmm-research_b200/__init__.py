"""esmm-research_b200: ctypes binding of libesmm_b200.so, the B200 (sm_100a) joint-sparse SGEMM.

The product is the C-ABI library (include/esmm.h) and the C++ driver / runner shim on top of it
(driver.cu, include/runners.cuh).  This module only loads the library and gives the tests and the
benchmark typed access to its entry points; it holds no compute of its own and has no CPU path:
if the library is missing, `lib()` raises.

The directory name has a hyphen, so load it with `__graft_entry__.load_package()` (importlib by
path) rather than a plain import statement.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libesmm_b200.so")
CHECKED_LIB_PATH = os.path.join(_HERE, "libesmm_b200_checked.so")
EXE_PATH = os.path.join(_HERE, "exec_b200")
HEADER_PATH = os.path.join(os.path.dirname(_HERE), "include", "esmm.h")

OK, ERR_NULL, ERR_SHAPE, ERR_ALIGN, ERR_CUDA, ERR_TIMEOUT, ERR_IO, ERR_UNSUPPORTED, ERR_VERIFY, \
    ERR_TOO_LARGE, ERR_MISMATCH, ERR_BOUNDS = range(12)


class EsmmError(RuntimeError):
    def __init__(self, status: int, where: str):
        L = lib()
        msg = L.esmm_strerror(status).decode()
        cuda = L.esmm_last_cuda_error().decode()
        super().__init__(f"{where}: {msg} (status {status})" + (f" [{cuda}]" if cuda else ""))
        self.status = status


class ABPatternMetadata(C.Structure):
    """Mirror of esmm_ab_pattern_metadata (the reference's ABPatternMetadata,
    src/preprocessors/ab_preprocessor.cu:7-17)."""
    _fields_ = [("d_a_patterns", C.c_void_p), ("d_b_patterns", C.c_void_p), ("owns_b_patterns", C.c_int),
                ("numMBlocks", C.c_int), ("numNBlocks", C.c_int), ("numKBlocks", C.c_int),
                ("a_sparsity", C.c_float), ("b_sparsity", C.c_float), ("joint_sparsity", C.c_float)]


_vp, _i, _f = C.c_void_p, C.c_int, C.c_float
_SIGNATURES = {
    "esmm_strerror": (C.c_char_p, [_i]),
    "esmm_last_cuda_error": (C.c_char_p, []),
    "esmm_version": (_i, []),
    "esmm_num_k_blocks": (_i, [_i]),
    "esmm_a_pattern_bytes": (C.c_size_t, [_i, _i, _i]),
    "esmm_b_pattern_bytes": (C.c_size_t, [_i, _i]),
    "esmm_pattern_from_string": (_i, [C.c_char_p]),
    "esmm_pattern_lut": (None, [C.c_uint8, C.POINTER(C.c_uint8), C.POINTER(C.c_uint8 * 8)]),
    "esmm_preprocess_a": (_i, [_vp, _i, _i, _i, _vp, _vp]),
    "esmm_preprocess_b": (_i, [_vp, _i, _i, _vp, _vp]),
    "esmm_preprocess_ab": (_i, [_vp, _vp, _i, _i, _i, _i, _vp, C.POINTER(ABPatternMetadata)]),
    "esmm_free_ab_pattern_metadata": (_i, [C.POINTER(ABPatternMetadata)]),
    "esmm_bpat_save": (_i, [C.c_char_p, _vp, _i, _i]),
    "esmm_bpat_load": (_i, [C.c_char_p, _vp, _i, _i]),
    "esmm_gemm_ab": (_i, [_i, _i, _i, _vp, _vp, _vp, _vp, _vp, _i, _vp]),
    "esmm_a_packed_bytes": (C.c_size_t, [_i, _i]),
    "esmm_preprocess_a_packed": (_i, [_vp, _i, _i, _vp, _vp, _vp]),
    "esmm_gemm_ab_packed": (_i, [_i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp]),
    "esmm_sgemm_joint_workspace_bytes": (C.c_size_t, [_i, _i]),
    "esmm_sgemm_joint": (_i, [_i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp]),
    "esmm_sgemm_joint_static": (_i, [_i, _i, _i, _vp, _vp, _vp, _vp, _vp]),
    "esmm_device_status": (_i, [_vp]),
    "esmm_tuning_set": (_i, [C.c_char_p, _i]),
    "esmm_tuning_reset": (None, []),
    "esmm_last_tiled_kernel_warps": (_i, []),
    "esmm_checked_build": (_i, []),
    "esmm_selftest_bounds_report": (_i, [_vp]),
    "esmm_selftest_bounded_wait": (_i, [C.c_uint, _vp]),
    "esmm_tf32x3_b_create": (_i, [_vp, _i, _i, _i, C.POINTER(_vp)]),
    "esmm_tf32x3_b_destroy": (None, [_vp]),
    "esmm_tf32x3_b_live_k": (_i, [_vp]),
    "esmm_tf32x3_workspace_bytes": (C.c_size_t, [_i, _i]),
    "esmm_sgemm_joint_tf32x3": (_i, [_i, _vp, _vp, _vp, _vp, _vp]),
    "esmm_cusparse_spmm": (_i, [_i, _i, _i, _vp, _vp, _vp, _i, C.POINTER(_f), C.POINTER(_f),
                                C.POINTER(C.c_longlong)]),
    "esmm_plan_create": (_i, [_i, _i, _i, _vp, _i, C.POINTER(_vp)]),
    "esmm_plan_run": (_i, [_vp, _vp, _vp]),
    "esmm_plan_submit": (_i, [_vp, _vp, _vp]),
    "esmm_plan_wait": (_i, [_vp]),
    "esmm_plan_destroy": (_i, [_vp]),
    "esmm_cublas_sgemm": (_i, [_i, _i, _i, _vp, _vp, _vp, _vp]),
    "esmm_ffma_peak_tflops": (_i, [C.POINTER(C.c_double), C.POINTER(_i)]),
    "esmm_fill_normal": (_i, [_vp, C.c_long, C.c_long, _i, C.c_uint64, _f, _f, _i, _i, C.c_uint8, _f, _i,
                              C.c_uint64, _vp]),
    "esmm_interleave_shards": (_i, [_vp, _vp, _i, _i, _i, _vp]),
    "esmm_randomize_matrix_with_pattern": (_i, [_vp, _i, _i, C.c_char_p]),
    "esmm_randomize_matrix_unstructured": (_i, [_vp, _i, _i, _f, C.c_uint]),
    "esmm_randomize_matrix_a_blocklevel": (_i, [_vp, _i, _i, _i, _i, _f, C.c_uint]),
    "esmm_randomize_matrix_b_blocklevel": (_i, [_vp, _i, _i, _i, _i, _f, C.c_uint]),
    "esmm_print_usage": (None, [C.c_char_p, _i]),
    "esmm_multi_shard_columns": (_i, [_i, _i, _i, C.POINTER(_i), C.POINTER(_i)]),
    "esmm_multi_create": (_i, [_i, _i, _i, _i, C.POINTER(_i), C.POINTER(_vp)]),
    "esmm_multi_num_gpus": (_i, [_vp]),
    "esmm_multi_upload": (_i, [_vp, _vp, _vp]),
    "esmm_multi_fill": (_i, [_vp, C.c_uint64, _i, C.c_uint8, C.c_uint8, _f, _f, _i]),
    "esmm_multi_run": (_i, [_vp, _i, C.POINTER(_f), C.POINTER(_f)]),
    "esmm_multi_download": (_i, [_vp, _vp]),
    "esmm_multi_gather": (_i, [_vp, _vp, C.POINTER(_f)]),
    "esmm_multi_gathered_c": (_vp, [_vp]),
    "esmm_multi_destroy": (_i, [_vp]),
    "esmm_skip_stats": (_i, [_vp, _vp, _i, _i, _i, _i, _i, _i, C.POINTER(C.c_longlong * 6)]),
    "esmm_kernel_id_valid": (_i, [_i]),
    "esmm_kernel_name": (C.c_char_p, [_i]),
    "esmm_parse_kernel_selection": (_i, [C.c_char_p, C.POINTER(_i), _i]),
    "esmm_run_kernel": (_i, [_i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, C.POINTER(_i),
                             C.POINTER(_f)]),
    "esmm_run_kernel_cached_b": (_i, [_i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp, C.POINTER(_i),
                                      C.POINTER(_f)]),
    "esmm_run_kernel_pattern": (_i, [_i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp, C.c_char_p,
                                     C.POINTER(_i), C.POINTER(_f)]),
}

_lib = None


def lib() -> C.CDLL:
    """The loaded C-ABI library.  Raises if it has not been built: there is no fallback."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: run `python esmm-research_b200/build.py` "
                               "(or __graft_entry__.build()); this package has no CPU or PyTorch fallback")
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def load_library(path: str) -> C.CDLL:
    """Another build of the same ABI (the bounds-checked one) with the typed signatures applied."""
    if not os.path.exists(path):
        raise RuntimeError(f"{path} is missing: run `python esmm-research_b200/build.py`")
    L = C.CDLL(path)
    for name, (res, args) in _SIGNATURES.items():
        fn = getattr(L, name)
        fn.restype = res
        fn.argtypes = args
    return L


def exported_names() -> list[str]:
    return sorted(_SIGNATURES)


def check(status: int, where: str) -> None:
    if status != OK:
        raise EsmmError(status, where)


# ---- thin typed helpers (device pointers are plain integers) -----------------------------------
def preprocess_a(d_A: int, M: int, K: int, d_out: int, tile_m: int = 32, stream: int = 0) -> None:
    check(lib().esmm_preprocess_a(d_A, M, K, tile_m, d_out, stream), "esmm_preprocess_a")


def preprocess_b(d_B: int, K: int, N: int, d_out: int, stream: int = 0) -> None:
    check(lib().esmm_preprocess_b(d_B, K, N, d_out, stream), "esmm_preprocess_b")


def gemm_ab(M, N, K, d_A, d_B, d_C, d_a_pat, d_b_pat, a_tile_m: int = 32, stream: int = 0) -> None:
    check(lib().esmm_gemm_ab(M, N, K, d_A, d_B, d_C, d_a_pat, d_b_pat, a_tile_m, stream), "esmm_gemm_ab")


def sgemm_joint(M, N, K, d_A, d_B, d_C, d_b_pat, d_workspace, stream: int = 0) -> None:
    """Packing preprocess of A + packed GEMM; d_workspace holds sgemm_joint_workspace_bytes(M, K)."""
    check(lib().esmm_sgemm_joint(M, N, K, d_A, d_B, d_C, d_b_pat, d_workspace, stream), "esmm_sgemm_joint")


def sgemm_joint_workspace_bytes(M: int, K: int) -> int:
    return int(lib().esmm_sgemm_joint_workspace_bytes(M, K))


def a_packed_bytes(M: int, K: int) -> int:
    return int(lib().esmm_a_packed_bytes(M, K))


def preprocess_a_packed(d_A: int, M: int, K: int, d_out: int, d_packed: int, stream: int = 0) -> None:
    check(lib().esmm_preprocess_a_packed(d_A, M, K, d_out, d_packed, stream), "esmm_preprocess_a_packed")


def gemm_ab_packed(M, N, K, d_a_packed, d_B, d_C, d_a_pat, d_b_pat, stream: int = 0) -> None:
    check(lib().esmm_gemm_ab_packed(M, N, K, d_a_packed, d_B, d_C, d_a_pat, d_b_pat, stream),
          "esmm_gemm_ab_packed")


class Tf32x3B:
    """The "B offline" state of the optional 3xTF32 tensor-core path (B patterns, kept k, B transposed and
    split), owned by the library; `compact` drops k whose row of B is all zero from both operands."""

    def __init__(self, d_B: int, K: int, N: int, compact: bool = True):
        self.handle = C.c_void_p()
        self.K, self.N = K, N
        check(lib().esmm_tf32x3_b_create(d_B, K, N, 1 if compact else 0, C.byref(self.handle)),
              "esmm_tf32x3_b_create")

    @property
    def live_k(self) -> int:
        return int(lib().esmm_tf32x3_b_live_k(self.handle))

    def close(self) -> None:
        if self.handle:
            lib().esmm_tf32x3_b_destroy(self.handle)
            self.handle = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def tf32x3_workspace_bytes(M: int, K: int) -> int:
    return int(lib().esmm_tf32x3_workspace_bytes(M, K))


def sgemm_joint_tf32x3(M: int, d_A: int, b: Tf32x3B, d_C: int, d_workspace: int, stream: int = 0) -> None:
    """Optional tensor-core variant (3xTF32; within a few 1e-6 of the FP32 path, not bit-identical): split of
    A + A patterns + product.  d_workspace holds tf32x3_workspace_bytes(M, b.K)."""
    check(lib().esmm_sgemm_joint_tf32x3(M, d_A, b.handle, d_C, d_workspace, stream), "esmm_sgemm_joint_tf32x3")


def device_status(stream: int = 0) -> None:
    check(lib().esmm_device_status(stream), "esmm_device_status")


def cublas_sgemm(M, N, K, d_A, d_B, d_C, stream: int = 0) -> None:
    check(lib().esmm_cublas_sgemm(M, N, K, d_A, d_B, d_C, stream), "esmm_cublas_sgemm")


def fill_normal(d_out, rows, cols, k_axis, seed, mean=0.0, std=1.0, relu=False, mode=0, pattern=0xFF,
                p_live=1.0, gran=32, seed2=0, stream: int = 0) -> None:
    check(lib().esmm_fill_normal(d_out, rows, cols, k_axis, seed, mean, std, int(relu), mode, pattern, p_live,
                                 gran, seed2, stream), "esmm_fill_normal")


def ffma_peak_tflops() -> tuple[float, int]:
    t, s = C.c_double(0), C.c_int(0)
    check(lib().esmm_ffma_peak_tflops(C.byref(t), C.byref(s)), "esmm_ffma_peak_tflops")
    return float(t.value), int(s.value)


def pattern_from_string(s: str) -> int:
    return lib().esmm_pattern_from_string(s.encode())


def parse_kernel_selection(s: str) -> list[int]:
    buf = (C.c_int * 32)()
    n = lib().esmm_parse_kernel_selection(s.encode(), buf, 32)
    return list(buf)[:max(0, min(n, 32))]
