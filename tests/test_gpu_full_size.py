"""GPU parity at the sizes the benchmark times: configs 3 (4096^3, independent 64-granular tile patterns), 4 (LLM MLP
shape, M = 2048 and M = 16) and one column shard of config 5 (16384 x 16384 x 2048).  Pattern bytes are compared in
full with the oracle; C is compared bit for bit with the oracle's FMA chain (src/kernels/esmm_ab_optimized_v3.cu:74-77,
157, 183-203 of the reference) on a sample of 32-row blocks that touches the first and the last block, both halves of a
64-row tile and every group of the kernel's tile raster.  These sizes exercise what the small cases do not: many
rounds of the grouped raster, 86-tile-wide rows, 2048 K blocks per list together with many tiles per CTA."""
import numpy as np
import pytest

import workloads

pytestmark = pytest.mark.gpu
TOL = 1e-4  # max |C - C_ref| / max |C_ref|; the observed difference is 0 (asserted as equal bits)


def sample_blocks(M: int) -> list[int]:
    """32-row blocks: first, its neighbour in the same 64-row tile, one inside every 1024-row raster group at a
    different offset each time, and the last one."""
    nb = -(-M // 32)
    picks = {0, min(1, nb - 1), nb - 1}
    for g, first in enumerate(range(0, nb, 32)):
        picks.add(min(nb - 1, first + (5 + 7 * g) % 32))
    return sorted(picks)


def check_problem(t, pkg, oracle, dA, dB, expect_a_bytes=None):
    """Whole per-call path on device-resident A, B: B patterns (offline step), packing preprocess + GEMM."""
    M, K = dA.shape
    N = dB.shape[1]
    bp = t.full((-(-N // 32), -(-K // 8)), 0xEE, dtype=t.uint8, device="cuda")
    pkg.preprocess_b(dB.data_ptr(), K, N, bp.data_ptr())
    ws = t.empty(pkg.sgemm_joint_workspace_bytes(M, K), dtype=t.uint8, device="cuda")
    ws.fill_(0xFF)                                        # whatever the packer leaves unwritten is a NaN pattern
    c = t.full((M, N), float("nan"), device="cuda")
    pkg.sgemm_joint(M, N, K, dA.data_ptr(), dB.data_ptr(), c.data_ptr(), bp.data_ptr(), ws.data_ptr())
    pkg.device_status()
    n_ap = -(-M // 32) * -(-K // 8)
    ap = ws[:n_ap].reshape(-(-M // 32), -(-K // 8)).cpu().numpy()
    A, B = dA.cpu().numpy(), dB.cpu().numpy()
    oap, obp = oracle.preprocess_a(A), oracle.preprocess_b(B)
    assert np.array_equal(ap, oap), "A pattern bytes differ from the oracle"
    assert np.array_equal(bp.cpu().numpy(), obp), "B pattern bytes differ from the oracle"
    if expect_a_bytes is not None:
        assert set(np.unique(oap)) == set(expect_a_bytes)
    assert not bool(t.isnan(c).any())
    for blk in sample_blocks(M):
        r0, r1 = blk * 32, min(M, blk * 32 + 32)
        want = oracle.gemm_joint(A[r0:r1], B, oap[blk:blk + 1], obp)
        got = c[r0:r1].cpu().numpy()
        assert oracle.rel_inf_err(got, want) <= TOL, blk
        assert np.array_equal(got, want), f"row block {blk}: not bit-identical to the oracle's FMA chain"
    return c, ap, bp


@pytest.mark.parametrize("pA,pB", [(0.5, 0.5), (0.3, 0.7), (0.2, 0.2)])
def test_config3_full_size(cuda, pkg, oracle_mod, pA, pB):
    """4096^3, for each 64-row block of A x 8-slice every K offset live with probability pA (B: 64 columns, pB)."""
    S = 4096
    dA = cuda.empty((S, S), device="cuda")
    dB = cuda.empty((S, S), device="cuda")
    pkg.fill_normal(dA.data_ptr(), S, S, 0, 11, mode=2, p_live=pA, gran=64, seed2=101)
    pkg.fill_normal(dB.data_ptr(), S, S, 1, 12, mode=2, p_live=pB, gran=64, seed2=102)
    _, ap, bp = check_problem(cuda, pkg, oracle_mod, dA, dB)
    # generator granularity 64 against pattern granularity 32: pattern rows come in identical pairs
    bpn = bp.cpu().numpy()
    assert np.array_equal(ap[0::2], ap[1::2]) and np.array_equal(bpn[0::2], bpn[1::2])
    dens = np.unpackbits(ap).mean(), np.unpackbits(bpn).mean()
    assert abs(dens[0] - pA) < 0.01 and abs(dens[1] - pB) < 0.01


@pytest.mark.parametrize("M", [2048, 16])
def test_config4_full_size(cuda, pkg, oracle_mod, M):
    """LLM MLP up-projection: K = 4096, N = 11008; A = pruned ReLU activations, B = block-pruned weights, one K-group
    permutation applied to both.  M = 16 takes the strip kernel, M = 2048 the tiled one (86 tiles per tile row)."""
    K, N = 4096, 11008
    A, B = workloads.llm_mlp(M, N, K, seed=40 + M)
    dA, dB = cuda.from_numpy(A).cuda(), cuda.from_numpy(B).cuda()
    _, ap, bp = check_problem(cuda, pkg, oracle_mod, dA, dB)
    assert 0.30 < (ap != 0).mean() < 0.50 and 0.40 < (bp.cpu().numpy() != 0).mean() < 0.60


def test_config5_one_shard_full_size(cuda, pkg, oracle_mod):
    """One of eight column shards of 16384^3 with the uniform pattern 11000000 (byte 0x03): K = 16384 is 2048 K blocks
    per list, 128 x 16 tiles on 148 CTAs."""
    S, W = 16384, 2048
    dA = cuda.empty((S, S), device="cuda")
    dB = cuda.empty((S, W), device="cuda")
    pkg.fill_normal(dA.data_ptr(), S, S, 0, 1, mode=1, pattern=0x03)
    pkg.fill_normal(dB.data_ptr(), S, W, 1, 1003, mode=1, pattern=0x03)
    c, ap, bp = check_problem(cuda, pkg, oracle_mod, dA, dB, expect_a_bytes={0x03})
    assert set(np.unique(bp.cpu().numpy())) == {0x03}
    # size-independent property on the whole shard: scaling A by a power of two scales C exactly
    dA *= 0.5
    ws = cuda.empty(pkg.sgemm_joint_workspace_bytes(S, S), dtype=cuda.uint8, device="cuda")
    c2 = cuda.empty_like(c)
    pkg.sgemm_joint(S, W, S, dA.data_ptr(), dB.data_ptr(), c2.data_ptr(), bp.data_ptr(), ws.data_ptr())
    pkg.device_status()
    assert cuda.equal(c2, c * 0.5)
