"""CPU tests of the C-ABI library: it loads without a GPU, exports every symbol include/esmm.h
declares, validates arguments before touching a device, and its host-side helpers (kernel-id
parser and names, pattern strings, skip statistics, B pattern cache file) match the reference."""
import ctypes as C
import os
import re

import numpy as np
import pytest

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def test_library_exports_every_declared_symbol(pkg):
    hdr = open(pkg.HEADER_PATH).read()
    hdr = re.sub(r"/\*.*?\*/", "", hdr, flags=re.S)
    declared = set(re.findall(r"\b(esmm_[a-z0-9_]+)\s*\(", hdr))
    assert len(declared) >= 30
    L = pkg.lib()
    for name in sorted(declared):
        assert hasattr(L, name), f"{name} is declared in esmm.h but not exported"
    assert declared == set(pkg.exported_names()), declared ^ set(pkg.exported_names())


def test_no_cpu_fallback_without_library(pkg, monkeypatch):
    monkeypatch.setattr(pkg, "_lib", None)
    monkeypatch.setattr(pkg, "LIB_PATH", "/nonexistent/libesmm_b200.so")
    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        pkg.lib()


def test_argument_validation_needs_no_device(pkg):
    L = pkg.lib()
    ok_ptr = 4096  # never dereferenced: validation fails first
    assert L.esmm_gemm_ab(128, 128, 128, 0, ok_ptr, ok_ptr, ok_ptr, ok_ptr, 32, 0) == pkg.ERR_NULL
    assert L.esmm_gemm_ab(128, 128, 130, ok_ptr, ok_ptr, ok_ptr, ok_ptr, ok_ptr, 32, 0) == pkg.ERR_SHAPE
    assert L.esmm_gemm_ab(128, 126, 128, ok_ptr, ok_ptr, ok_ptr, ok_ptr, ok_ptr, 32, 0) == pkg.ERR_SHAPE
    assert L.esmm_gemm_ab(0, 128, 128, ok_ptr, ok_ptr, ok_ptr, ok_ptr, ok_ptr, 32, 0) == pkg.ERR_SHAPE
    assert L.esmm_gemm_ab(128, 128, 128, ok_ptr + 4, ok_ptr, ok_ptr, ok_ptr, ok_ptr, 32, 0) == pkg.ERR_ALIGN
    assert L.esmm_gemm_ab(128, 128, 128, ok_ptr, ok_ptr, ok_ptr, ok_ptr, ok_ptr, 48, 0) == pkg.ERR_UNSUPPORTED
    assert L.esmm_gemm_ab_packed(128, 128, 128, ok_ptr, ok_ptr, 0, ok_ptr, ok_ptr, 0) == pkg.ERR_NULL
    assert L.esmm_gemm_ab_packed(128, 128, 2, ok_ptr, ok_ptr, ok_ptr, ok_ptr, ok_ptr, 0) == pkg.ERR_SHAPE
    assert L.esmm_preprocess_a(0, 32, 32, 32, ok_ptr, 0) == pkg.ERR_NULL
    assert L.esmm_preprocess_a(ok_ptr, 32, 0, 32, ok_ptr, 0) == pkg.ERR_SHAPE
    assert L.esmm_preprocess_a_packed(ok_ptr, 32, 34, ok_ptr, ok_ptr, 0) == pkg.ERR_SHAPE
    assert L.esmm_preprocess_b(ok_ptr, 32, 32, 0, 0) == pkg.ERR_NULL
    assert L.esmm_sgemm_joint(128, 128, 128, ok_ptr, ok_ptr, ok_ptr, ok_ptr, 0, 0) == pkg.ERR_NULL
    assert L.esmm_sgemm_joint(128, 128, 128, ok_ptr, ok_ptr, ok_ptr, ok_ptr, ok_ptr + 16, 0) == pkg.ERR_ALIGN
    assert L.esmm_run_kernel(29, 128, 128, 128, 0, 0, 0, 0, 0, 1, 0, 0, None, None) == pkg.ERR_NULL
    assert L.esmm_run_kernel(33, 128, 128, 128, ok_ptr, ok_ptr, ok_ptr, 0, 0, 1, 0, 0, None, None) == pkg.ERR_UNSUPPORTED
    assert L.esmm_run_kernel_pattern(14, 128, 128, 128, ok_ptr, ok_ptr, ok_ptr, 0, 0, 1, 0, 0, None, b"1111", None,
                                     None) == pkg.ERR_SHAPE
    assert L.esmm_interleave_shards(ok_ptr, ok_ptr, 8, 12, 2, 0) == pkg.ERR_SHAPE
    for st in range(12):
        assert L.esmm_strerror(st)


def test_geometry(pkg):
    L = pkg.lib()
    assert L.esmm_num_k_blocks(4096) == 512 and L.esmm_num_k_blocks(20) == 3
    assert L.esmm_a_pattern_bytes(4096, 4096, 32) == 128 * 512
    assert L.esmm_a_pattern_bytes(100, 20, 32) == 4 * 3
    assert L.esmm_b_pattern_bytes(4096, 11008) == 344 * 512
    assert L.esmm_a_packed_bytes(4096, 4096) == 4096 * 4096 * 4
    assert L.esmm_a_packed_bytes(100, 20) == 128 * 24 * 4
    ws = L.esmm_sgemm_joint_workspace_bytes(4096, 4096)
    assert ws == 128 * 512 + 4096 * 4096 * 4


def test_pattern_string_and_lut_match_oracle(pkg, oracle_mod):
    L = pkg.lib()
    for s in ("11111111", "11110000", "11000000", "10000000", "01010101", "1111000", "1111000x"):
        assert pkg.pattern_from_string(s) == oracle_mod.pattern_from_string(s)
    for p in range(256):
        cnt = C.c_uint8(0)
        off = (C.c_uint8 * 8)()
        L.esmm_pattern_lut(p, C.byref(cnt), C.byref(off))
        assert (int(cnt.value), list(off)) == oracle_mod.pattern_lut(p)


def test_kernel_selection_and_names_match_reference(pkg):
    g = np.load(os.path.join(GOLD, "ref_cpu.npz"))
    L = pkg.lib()
    for sel, parsed in zip(g["selections"], g["parsed"]):
        want = [int(x) for x in str(parsed).split(",") if x]
        assert pkg.parse_kernel_selection(str(sel)) == want, sel
    assert pkg.parse_kernel_selection("abc") == [] and pkg.parse_kernel_selection("") == []
    for i, name in zip(g["name_ids"], g["names"]):
        assert L.esmm_kernel_name(int(i)).decode() == str(name)
    valid = [i for i in range(40) if L.esmm_kernel_id_valid(i)]
    assert valid == [14, 15, 16, 17, 20, 21, 25, 26, 27, 28, 29, 30]
    # additive id outside the reference's 1-100 range: the optional tensor-core variant; 'all' does not select it
    assert L.esmm_kernel_id_valid(129) and b"3xTF32" in L.esmm_kernel_name(129)
    assert pkg.parse_kernel_selection("129") == [129] and 129 not in pkg.parse_kernel_selection("all")


def test_skip_stats_match_oracle(pkg, oracle_mod):
    rng = np.random.default_rng(0)
    for (nmb, nnb, nkb, wm, wn) in [(8, 8, 16, 2, 4), (4, 8, 5, 1, 4), (6, 6, 9, 3, 2)]:
        a = rng.integers(0, 256, (nmb, nkb), dtype=np.uint8) & rng.integers(0, 256, (nmb, nkb), dtype=np.uint8)
        b = rng.integers(0, 256, (nnb, nkb), dtype=np.uint8) & rng.integers(0, 256, (nnb, nkb), dtype=np.uint8)
        a[rng.random(a.shape) < 0.3] = 0
        out = (C.c_longlong * 6)()
        st = pkg.lib().esmm_skip_stats(a.ctypes.data, b.ctypes.data, nmb // wm, nnb // wn, nkb, wm, wn, 8,
                                       C.byref(out))
        assert st == 0
        want = oracle_mod.skip_stats(a, b, wm, wn)
        assert list(out) == [want[k] for k in ("block_skips", "total_k", "warp_skips", "total_warp_k",
                                               "dot_skips", "total_dot")]


def test_b_pattern_cache_round_trip(pkg, tmp_path):
    L = pkg.lib()
    K, N = 72, 132
    n = L.esmm_b_pattern_bytes(K, N)
    pat = np.random.default_rng(1).integers(0, 256, n, dtype=np.uint8)
    path = str(tmp_path / "w.bpat").encode()
    assert L.esmm_bpat_save(path, pat.ctypes.data, K, N) == 0
    back = np.zeros(n, np.uint8)
    assert L.esmm_bpat_load(path, back.ctypes.data, K, N) == 0
    assert np.array_equal(back, pat)
    assert L.esmm_bpat_load(path, back.ctypes.data, K, N + 32) == pkg.ERR_MISMATCH
    assert L.esmm_bpat_load(path, back.ctypes.data, K + 8, N) == pkg.ERR_MISMATCH
    assert L.esmm_bpat_load(str(tmp_path / "missing").encode(), back.ctypes.data, K, N) == pkg.ERR_IO
    with open(tmp_path / "w.bpat", "ab") as f:
        f.write(b"x")
    assert L.esmm_bpat_load(path, back.ctypes.data, K, N) == pkg.ERR_IO
    (tmp_path / "junk").write_bytes(b"not a pattern file at all, but long enough for a header")
    assert L.esmm_bpat_load(str(tmp_path / "junk").encode(), back.ctypes.data, K, N) == pkg.ERR_IO


def test_compute_entry_points_fail_loudly_without_gpu(pkg):
    """No CPU fallback: on a machine without a CUDA device the compute calls report ESMM_ERR_CUDA."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    a = np.zeros((32, 32), np.float32)
    out = np.zeros(4, np.uint8)
    assert pkg.lib().esmm_preprocess_a(a.ctypes.data, 32, 32, 32, out.ctypes.data, 0) == pkg.ERR_CUDA
    assert pkg.lib().esmm_last_cuda_error()


def test_tf32x3_host_side_without_gpu(pkg):
    """The parts of the optional tensor-core entry points that need no device: sizes and NULL handling."""
    import ctypes as C
    L = pkg.lib()
    assert L.esmm_tf32x3_workspace_bytes(0, 64) == 0 and L.esmm_tf32x3_workspace_bytes(64, -8) == 0
    M, K = 100, 72
    pat = (int(L.esmm_a_pattern_bytes(M, K, 32)) + 255) & ~255
    assert L.esmm_tf32x3_workspace_bytes(M, K) == pat + 2 * M * K * 4
    assert L.esmm_tf32x3_b_live_k(None) == 0
    L.esmm_tf32x3_b_destroy(None)
    h = C.c_void_p()
    assert L.esmm_tf32x3_b_create(None, 64, 64, 1, C.byref(h)) == 1 and not h.value          # ESMM_ERR_NULL before any CUDA call
    assert L.esmm_sgemm_joint_tf32x3(32, None, None, None, None, None) == 1



def test_tuning_hooks_are_explicit_not_environment(pkg, monkeypatch):
    """Hooks are set by name through the C ABI; unknown names are refused; the environment is not consulted
    (no source file of the library calls getenv)."""
    import glob
    L = pkg.lib()
    assert L.esmm_tuning_set(b"TILE_M", 64) == 0 and L.esmm_tuning_set(b"TF32_PAIR", 0) == 0
    assert L.esmm_tuning_set(b"NO_SUCH_HOOK", 1) == pkg.ERR_UNSUPPORTED and L.esmm_tuning_set(None, 1) == pkg.ERR_UNSUPPORTED
    L.esmm_tuning_reset()
    csrc = os.path.join(os.path.dirname(pkg.LIB_PATH), "csrc")
    for path in glob.glob(os.path.join(csrc, "*")):
        assert "getenv" not in open(path).read(), path


def test_multi_gpu_host_side_validation(pkg):
    """The sharded entry points validate on the host before touching a device (or NCCL)."""
    import ctypes as C
    L = pkg.lib()
    n0, n1 = C.c_int(-1), C.c_int(-1)
    assert L.esmm_multi_shard_columns(16384, 8, 3, C.byref(n0), C.byref(n1)) == 0 and (n0.value, n1.value) == (6144, 8192)
    assert L.esmm_multi_shard_columns(4096, 3, 0, None, None) == pkg.ERR_SHAPE        # not whole tiles per shard
    assert L.esmm_multi_shard_columns(4096, 2, 2, None, None) == pkg.ERR_SHAPE        # rank out of range
    assert L.esmm_multi_shard_columns(4096, 0, 0, None, None) == pkg.ERR_SHAPE
    h = C.c_void_p()
    assert L.esmm_multi_create(256, 4096, 256, 3, None, C.byref(h)) == pkg.ERR_SHAPE and not h.value
    assert L.esmm_multi_create(256, 256, 258, 2, None, C.byref(h)) == pkg.ERR_SHAPE
    assert L.esmm_multi_create(256, 256, 256, 2, None, None) == pkg.ERR_NULL
    assert L.esmm_multi_run(None, 1, None, None) == pkg.ERR_NULL and L.esmm_multi_gather(None, None, None) == pkg.ERR_NULL
    assert L.esmm_multi_download(None, None) == pkg.ERR_NULL and L.esmm_multi_destroy(None) == 0
    assert L.esmm_multi_num_gpus(None) == 0 and not L.esmm_multi_gathered_c(None)
