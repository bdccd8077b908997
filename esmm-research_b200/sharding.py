"""N-column sharding of C = A * B across the GPUs of one box (host-side logic only).

The reference has no multi-GPU code.  The joint-sparse SGEMM partitions without any exchange:
rank g owns columns [n0, n1) of B, of the B patterns and of C; A and its patterns are replicated,
and every rank runs the A preprocessor on its own replica.  A collective appears only at the two
ends: when A arrives from host memory (`upload_rows_replicated`: every rank copies 1 / world of the
rows over its own PCIe link and the replicas are completed by an all-gather over NVLink, instead of
`world` full copies competing for host memory bandwidth) and when the caller wants all of C on one
rank (`gather_columns`).

Nothing here computes: the compute calls are the C-ABI entry points, made by the caller on its
shard.  torch.distributed (NCCL on GPUs, gloo in the CPU tests) is the only dependency.
"""
from __future__ import annotations

from dataclasses import dataclass

PATTERN_COLS = 32  # columns per B pattern byte: a shard boundary must not split a pattern block


@dataclass(frozen=True)
class ColumnShard:
    rank: int
    world: int
    N: int
    n0: int
    n1: int

    @property
    def width(self) -> int:
        return self.n1 - self.n0


def shard_columns(N: int, world: int, rank: int, align: int = 128) -> ColumnShard:
    """Contiguous, equal column blocks.  Equal widths keep the gather a plain all-gather; `align`
    (default: the GEMM tile width) keeps every shard a whole number of tiles and pattern blocks."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError(f"bad rank {rank} of {world}")
    if align % PATTERN_COLS:
        raise ValueError("align must be a multiple of the 32-column pattern block")
    if N % (world * align):
        raise ValueError(f"N = {N} does not split into {world} shards of a multiple of {align} columns")
    w = N // world
    return ColumnShard(rank, world, N, rank * w, (rank + 1) * w)


def preflight(ok: bool, dist, device=None) -> bool:
    """All ranks learn, before any launch or data collective, whether every rank is ready
    (buffers allocated, library loaded, shapes valid).  Returns True only if all are."""
    import torch
    flag = torch.tensor([1 if ok else 0], dtype=torch.int32, device=device)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    return bool(flag.item() == 1)


def max_over_ranks(value: float, dist, device=None) -> float:
    """Whole-job time of a step = the slowest rank's device time."""
    import torch
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def row_slice(M: int, world: int, rank: int) -> tuple[int, int]:
    """Rows [r0, r1) of A that rank `rank` brings in from host memory: equal slices (the all-gather is
    a plain one), which needs M % world == 0."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError(f"bad rank {rank} of {world}")
    if M % world:
        raise ValueError(f"M = {M} does not split into {world} equal row slices")
    rows = M // world
    return rank * rows, (rank + 1) * rows


def upload_rows_replicated(h_rows, d_full, rank: int, world: int, dist) -> None:
    """Makes d_full ([M, K], this rank's device replica of A) complete on every rank from host slices.

    h_rows: this rank's rows [r0, r1) of A in (pinned) host memory, r0, r1 = row_slice(M, world, rank).
    The slice is copied into its place in d_full and the other ranks' slices arrive by an in-place
    all-gather.  Work on the current stream of d_full's device; with world == 1 it is a plain copy."""
    M = d_full.shape[0]
    r0, r1 = row_slice(M, world, rank)
    if tuple(h_rows.shape) != (r1 - r0, d_full.shape[1]):
        raise ValueError(f"host slice has shape {tuple(h_rows.shape)}, expected {(r1 - r0, d_full.shape[1])}")
    mine = d_full[r0:r1]
    mine.copy_(h_rows, non_blocking=True)
    if world > 1:
        dist.all_gather_into_tensor(d_full.view(-1), mine.view(-1))


def gather_columns(c_shard, shard: ColumnShard, dist, interleave=None):
    """All-gathers the [M, width] shards and returns the row-major [M, N] matrix (on every rank).

    `interleave(staging, out, M, N, world)` turns the gathered [world, M, width] staging buffer
    into [M, N]; on GPUs pass the C-ABI's esmm_interleave_shards, the default is a torch permute."""
    import torch
    M = c_shard.shape[0]
    staging = torch.empty((shard.world, M, shard.width), dtype=c_shard.dtype, device=c_shard.device)
    dist.all_gather_into_tensor(staging.view(-1), c_shard.contiguous().view(-1))
    if interleave is None:
        return staging.permute(1, 0, 2).reshape(M, shard.N).contiguous()
    out = torch.empty((M, shard.N), dtype=c_shard.dtype, device=c_shard.device)
    interleave(staging, out, M, shard.N, shard.world)
    return out
