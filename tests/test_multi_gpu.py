"""Two GPUs: N-column shards must equal the single-GPU result bit for bit, through both host paths -
(1) one process per GPU over torch.distributed (NCCL): A assembled on every rank from per-rank row uploads, shards
    computed through the C ABI, gathered and interleaved;
(2) the C++ launcher of the library (esmm_multi_*, what `exec_b200 --gpus` runs): one process, one host thread per
    GPU, NCCL all-gather of C inside the library, and the CLI itself.
Skipped on a box with fewer than two GPUs; the host logic is also covered without GPUs by tests/test_sharding_cpu.py
and the launcher with both ranks on one device by tests/test_gpu_parity.py."""
import subprocess
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, results):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import importlib
    import torch
    import torch.distributed as dist
    import __graft_entry__ as g
    import workloads
    pkg = g.load_package()
    sharding = importlib.import_module("esmm_research_b200.sharding")
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        M, N, K = 256, 1024, 512
        A, B = workloads.tile_random(M, N, K, 0.5, 0.5, seed=5, gran_a=32, gran_b=32)
        sh = sharding.shard_columns(N, world, rank)

        def joint(Bm):
            n = Bm.shape[1]
            dA, dB = torch.from_numpy(A).cuda(), torch.from_numpy(np.ascontiguousarray(Bm)).cuda()
            bp = torch.empty(pkg.lib().esmm_b_pattern_bytes(K, n), dtype=torch.uint8, device="cuda")
            pkg.preprocess_b(dB.data_ptr(), K, n, bp.data_ptr())
            ws = torch.empty(pkg.sgemm_joint_workspace_bytes(M, K), dtype=torch.uint8, device="cuda")
            c = torch.empty((M, n), device="cuda")
            pkg.sgemm_joint(M, n, K, dA.data_ptr(), dB.data_ptr(), c.data_ptr(), bp.data_ptr(), ws.data_ptr())
            pkg.device_status()
            return c

        ok = sharding.preflight(True, dist, torch.device("cuda", rank))
        # A from host memory: each rank uploads its rows, the all-gather completes every replica
        r0, r1 = sharding.row_slice(M, world, rank)
        replica = torch.full((M, K), float("nan"), device="cuda")
        sharding.upload_rows_replicated(torch.from_numpy(A[r0:r1].copy()).pin_memory(), replica, rank, world, dist)
        torch.cuda.synchronize()
        ok = ok and torch.equal(replica.cpu(), torch.from_numpy(A))
        c_shard = joint(B[:, sh.n0:sh.n1])

        def interleave(staging, out, m, n, w):
            pkg.check(pkg.lib().esmm_interleave_shards(staging.data_ptr(), out.data_ptr(), m, n, w, 0), "interleave")

        full = sharding.gather_columns(c_shard, sh, dist, interleave)
        full2 = sharding.gather_columns(c_shard, sh, dist)          # torch permute path
        torch.cuda.synchronize()
        want = joint(B)
        results[rank] = bool(ok and torch.equal(full, want) and torch.equal(full2, want))
    finally:
        dist.destroy_process_group()


@pytest.mark.gpu
def test_two_gpu_column_shards_match_single_gpu(cuda):
    if cuda.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_worker, args=(2, 29650 + os.getpid() % 300, results), nprocs=2, join=True)
    assert dict(results) == {0: True, 1: True}


_LAUNCHER_CHILD = r"""
import ctypes as C, sys
import numpy as np
sys.path.insert(0, {root!r}); sys.path.insert(0, {root!r} + "/tests")
import torch
import __graft_entry__ as g, workloads
pkg = g.load_package(); L = pkg.lib()
M, N, K = 384, 1024, 1024
A, B = workloads.tile_random(M, N, K, 0.4, 0.6, seed=7, gran_a=32, gran_b=32)
torch.cuda.set_device(0)
dA, dB = torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda()
bp = torch.empty(L.esmm_b_pattern_bytes(K, N), dtype=torch.uint8, device="cuda")
pkg.preprocess_b(dB.data_ptr(), K, N, bp.data_ptr())
ws = torch.empty(pkg.sgemm_joint_workspace_bytes(M, K), dtype=torch.uint8, device="cuda")
want = torch.empty((M, N), device="cuda")
pkg.sgemm_joint(M, N, K, dA.data_ptr(), dB.data_ptr(), want.data_ptr(), bp.data_ptr(), ws.data_ptr())
pkg.device_status()
want = want.cpu().numpy()
h = C.c_void_p()
pkg.check(L.esmm_multi_create(M, N, K, 2, None, C.byref(h)), "create")
pkg.check(L.esmm_multi_upload(h, A.ctypes.data, B.ctypes.data), "upload")
ms, per = C.c_float(0), (C.c_float * 2)()
pkg.check(L.esmm_multi_run(h, 2, C.byref(ms), per), "run")
down = np.full((M, N), np.nan, np.float32)
pkg.check(L.esmm_multi_download(h, down.ctypes.data), "download")
gath = np.full((M, N), np.nan, np.float32)
gms = C.c_float(0)
pkg.check(L.esmm_multi_gather(h, gath.ctypes.data, C.byref(gms)), "gather")
pkg.check(L.esmm_multi_gather(h, gath.ctypes.data, C.byref(gms)), "gather again")   # communicators are kept
assert L.esmm_multi_gathered_c(h)
L.esmm_multi_destroy(h)
print("RESULT", bool(np.array_equal(down, want)), bool(np.array_equal(gath, want)), per[0] > 0 and per[1] > 0, gms.value > 0)
"""


@pytest.mark.gpu
def test_cpp_launcher_two_gpus_matches_single_gpu(cuda, pkg):
    """esmm_multi_* on devices 0 and 1, in a child process with NVLS off: download and NCCL gather both give the
    single-GPU C bit for bit."""
    if cuda.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-c", _LAUNCHER_CHILD.format(root=ROOT)], capture_output=True, text=True, timeout=600,
                       env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    assert "RESULT True True True True" in r.stdout, r.stdout[-2000:]


@pytest.mark.gpu
def test_cli_gpus_2_gather(cuda, pkg):
    """`exec_b200 29 2 --gpus 2 --gather`: sharded run, C collected on GPU 0 over NCCL, verified against cuBLAS."""
    if cuda.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    for extra in (["--gather"], []):
        r = subprocess.run([pkg.EXE_PATH, "29", "2", "--gpus", "2", "--uniform", "--pattern", "11110000", "--size", "1024",
                            "--cpu-check", *extra], capture_output=True, text=True, timeout=600, env=env)
        out = r.stdout + r.stderr
        assert r.returncode == 0, out
        assert "2 GPUs, column shards of 512" in out and "PASSED" in out and "CPU SGEMM check" in out
        assert ("gather of C to GPU 0" in out) == bool(extra)
