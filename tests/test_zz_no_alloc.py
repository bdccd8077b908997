"""The allocation-free entry point, esmm_sgemm_joint_static, against esmm_sgemm_joint.

Some callers of the library can neither allocate device memory at call time nor pass a workspace
(an inference runtime that forbids allocation inside an operator's execute step, a process whose
allocator already owns the whole GPU).  For them the scratch of the per-call path lives in a fixed
array inside the library.  This file is collected last on purpose: if the entry point breaks, a run
that stops at the first failure has already run every other test.
"""
import numpy as np
import pytest

import workloads

TOL = 1e-4  # same bound as the other parity tests; the two entry points are in fact bit-identical


def _both(cuda, pkg, A, B, expect_no_driver_allocation):
    M, K = A.shape
    N = B.shape[1]
    dA, dB = cuda.from_numpy(A).cuda(), cuda.from_numpy(B).cuda()
    bp = cuda.empty(pkg.lib().esmm_b_pattern_bytes(K, N), dtype=cuda.uint8, device="cuda")
    pkg.preprocess_b(dB.data_ptr(), K, N, bp.data_ptr())
    ws = cuda.empty(pkg.sgemm_joint_workspace_bytes(M, K), dtype=cuda.uint8, device="cuda")
    want = cuda.full((M, N), float("nan"), device="cuda")
    pkg.sgemm_joint(M, N, K, dA.data_ptr(), dB.data_ptr(), want.data_ptr(), bp.data_ptr(), ws.data_ptr())
    pkg.device_status()
    got = cuda.full((M, N), float("nan"), device="cuda")
    cuda.cuda.synchronize()
    before = cuda.cuda.memory_allocated()
    free_before = cuda.cuda.mem_get_info()[0]      # cudaMemGetInfo: sees every allocation on the device, not only torch's
    pkg.check(pkg.lib().esmm_sgemm_joint_static(M, N, K, dA.data_ptr(), dB.data_ptr(), got.data_ptr(),
                                                bp.data_ptr(), None), "esmm_sgemm_joint_static")
    pkg.device_status()
    assert cuda.cuda.memory_allocated() == before
    if expect_no_driver_allocation:
        # the first call on a device may still load the library's device code (which is when the driver sets the
        # static array aside); from the second call on the device's free memory must not move at all
        assert cuda.cuda.mem_get_info()[0] == free_before
    return got.cpu().numpy(), want.cpu().numpy()


@pytest.mark.gpu
def test_static_scratch_entry_matches_workspace_entry_twice(cuda, pkg, oracle_mod):
    # first call: a larger, denser problem; second call: smaller and sparser, so that stale pattern
    # bytes and stale packed rows of the first call lie all around what the second one writes
    A1, B1 = workloads.tile_random(512, 384, 1024, 0.7, 0.6, seed=51, gran_a=32, gran_b=32)
    A2, B2 = workloads.tile_random(160, 256, 264, 0.2, 0.5, seed=52, gran_a=32, gran_b=32)
    for call, (A, B) in enumerate(((A1, B1), (A2, B2), (A1, B1))):
        got, want = _both(cuda, pkg, A, B, expect_no_driver_allocation=call > 0)
        assert not np.isnan(got).any()
        assert oracle_mod.rel_inf_err(got, want) <= TOL
        assert np.array_equal(got, want)
        assert np.array_equal(got, oracle_mod.gemm_joint(A, B))


def test_static_scratch_entry_rejects_oversized_problems(pkg):
    L = pkg.lib()
    p = 4096  # never dereferenced: the size check comes first
    assert L.esmm_sgemm_joint_static(4096, 4096, 4096, p, p, p, p, None) == pkg.ERR_TOO_LARGE
    assert b"static" in L.esmm_last_cuda_error() and b"4096 x 4096" in L.esmm_last_cuda_error()
    assert L.esmm_sgemm_joint_static(32, 128, 1 << 20, p, p, p, p, None) == pkg.ERR_TOO_LARGE  # pattern bytes
    assert L.esmm_sgemm_joint_static(128, 128, 128, 0, p, p, p, None) == pkg.ERR_NULL
    assert L.esmm_sgemm_joint_static(128, 128, 130, p, p, p, p, None) == pkg.ERR_SHAPE
