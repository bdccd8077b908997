"""CPU tests of the multi-GPU host logic: world_size 2 over gloo, one process per rank.  The ranks
compute their C shard with the oracle (this is a test of the partitioning and of the gather, not of
the kernels) and must reproduce the unsharded result bit for bit."""
import os
import sys

import numpy as np
import pytest
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, fail_rank, results):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import torch
    import torch.distributed as dist
    import __graft_entry__ as g
    import oracle
    import workloads
    g.load_package()
    import importlib
    sharding = importlib.import_module("esmm_research_b200.sharding")
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        M, N, K = 64, 512, 128
        A, B = workloads.tile_random(M, N, K, 0.5, 0.5, seed=3, gran_a=32, gran_b=32)  # same on every rank
        sh = sharding.shard_columns(N, world, rank)
        ready = sharding.preflight(rank != fail_rank, dist)
        if not ready:
            results[rank] = "aborted"
            return
        # A arrives from "host memory" in row slices, one per rank, and every rank ends with the whole of it
        r0, r1 = sharding.row_slice(M, world, rank)
        replica = torch.full((M, K), float("nan"))
        sharding.upload_rows_replicated(torch.from_numpy(A[r0:r1].copy()), replica, rank, world, dist)
        assert np.array_equal(replica.numpy(), A)
        A = replica.numpy()
        Bs = np.ascontiguousarray(B[:, sh.n0:sh.n1])                 # contiguous K x N/G shard
        bp = oracle.preprocess_b(Bs)                                  # per-shard cached B patterns
        assert np.array_equal(bp, oracle.preprocess_b(B)[sh.n0 // 32:sh.n1 // 32])
        Cs = oracle.gemm_joint(A, Bs, None, bp)
        full = sharding.gather_columns(torch.from_numpy(Cs), sh, dist).numpy()
        t = sharding.max_over_ranks(float(rank + 1), dist)
        ok = np.array_equal(full, oracle.gemm_joint(A, B)) and t == float(world)
        results[rank] = "ok" if ok else "mismatch"
    finally:
        dist.destroy_process_group()


def _run(world, fail_rank):
    mgr = mp.Manager()
    results = mgr.dict()
    port = 29500 + (os.getpid() % 2000) + (7 if fail_rank is not None else 0)
    mp.spawn(_worker, args=(world, port, fail_rank, results), nprocs=world, join=True)
    return dict(results)


def test_two_rank_shards_reproduce_unsharded_result():
    assert _run(2, None) == {0: "ok", 1: "ok"}


def test_preflight_failure_aborts_all_ranks_before_compute():
    assert _run(2, 1) == {0: "aborted", 1: "aborted"}


def test_shard_columns_validation():
    sys.path.insert(0, ROOT)
    import __graft_entry__ as g
    g.load_package()
    import importlib
    sharding = importlib.import_module("esmm_research_b200.sharding")
    s = [sharding.shard_columns(16384, 8, r) for r in range(8)]
    assert [x.width for x in s] == [2048] * 8 and s[0].n0 == 0 and s[7].n1 == 16384
    assert all(a.n1 == b.n0 for a, b in zip(s, s[1:]))
    with pytest.raises(ValueError):
        sharding.shard_columns(4096 + 128, 8, 0)
    with pytest.raises(ValueError):
        sharding.shard_columns(4096, 8, 8)
    with pytest.raises(ValueError):
        sharding.shard_columns(4096, 4, 0, align=48)
    assert [sharding.row_slice(4096, 4, r) for r in range(4)] == [(0, 1024), (1024, 2048), (2048, 3072), (3072, 4096)]
    with pytest.raises(ValueError):
        sharding.row_slice(4097, 4, 0)
    import torch
    full = torch.zeros((8, 4))
    sharding.upload_rows_replicated(torch.ones((8, 4)), full, 0, 1, None)      # one rank: a plain copy
    assert bool((full == 1).all())
    with pytest.raises(ValueError):
        sharding.upload_rows_replicated(torch.ones((4, 4)), full, 0, 1, None)
