"""Two ranks on two GPUs (NCCL): A assembled on every rank from per-rank row uploads, N-column shards computed
through the C ABI, gathered and interleaved, must equal the single-GPU result bit for bit.  Skipped on a box with fewer than two GPUs; the host
logic is also covered without GPUs by tests/test_sharding_cpu.py."""
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
