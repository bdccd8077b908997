"""Seeded synthetic inputs with the shapes, zero structures and value distributions of the
benchmark configurations (host side, numpy).  They stand in for the reference's rand()-based
generators and for the real LLM weights its scripts load, neither of which travel.

Every generator returns float32 row-major (A [M, K], B [K, N]); zeros are exactly 0.0.
"""
from __future__ import annotations

import numpy as np

PATTERNS = {"11111111": 0xFF, "11110000": 0x0F, "11000000": 0x03, "10000000": 0x01}


def pattern_byte(s: str) -> int:
    """String position i is K offset i is bit i ("11110000" -> 0x0F)."""
    assert len(s) == 8 and set(s) <= {"0", "1"}
    return sum(1 << i for i, c in enumerate(s) if c == "1")


def uniform_pattern(M, N, K, pattern: int, seed: int = 0):
    """Configs 1, 2, 5: N(0,1) values; in every 8-slice of K the offsets whose pattern bit is
    clear are zeroed in A's columns and in B's rows.  Seeds: seed for A, seed + 1 for B."""
    A = np.random.default_rng(seed).standard_normal((M, K), dtype=np.float32)
    B = np.random.default_rng(seed + 1).standard_normal((K, N), dtype=np.float32)
    live = np.array([(pattern >> (k & 7)) & 1 for k in range(K)], dtype=np.float32)
    A *= live[None, :]
    B *= live[:, None]
    return A, B


def tile_random(M, N, K, pA: float, pB: float, seed: int = 0, gran_a: int = 64, gran_b: int = 64):
    """Config 3: for each (gran_a-row block of A, 8-slice) each K offset is live with
    probability pA; for each (gran_b-column block of B, 8-slice) with probability pB."""
    rng = np.random.default_rng(seed)
    A = rng.standard_normal((M, K), dtype=np.float32)
    B = rng.standard_normal((K, N), dtype=np.float32)
    nkb = -(-K // 8)
    la = rng.random((-(-M // gran_a), nkb * 8)) < pA
    lb = rng.random((-(-N // gran_b), nkb * 8)) < pB
    A *= np.repeat(la, gran_a, axis=0)[:M, :K]
    B *= np.repeat(lb, gran_b, axis=0)[:N, :K].T
    return A, B


def llm_mlp(M, N, K, seed: int = 0, a_zero_frac: float = 0.6, b_keep_frac: float = 0.5):
    """Config 4: A = ReLU(N(0,1)) with whole 8-column groups per 32-row block zeroed where the
    group's L1 norm is below the a_zero_frac quantile; B = N(0, 0.02^2), per (8 K rows x 64
    columns) group L1-magnitude pruned to b_keep_frac; a seeded permutation of the K groups is
    applied to A's column groups and B's row groups alike (group granularity, so the 8-aligned
    zero groups survive)."""
    rng = np.random.default_rng(seed)
    A = np.maximum(rng.standard_normal((M, K), dtype=np.float32), 0.0)
    B = (0.02 * rng.standard_normal((K, N))).astype(np.float32)
    nkb = K // 8
    mb = -(-M // 32)
    Ap = np.zeros((mb * 32, K), np.float32)
    Ap[:M] = A
    l1a = np.abs(Ap).reshape(mb, 32, nkb, 8).sum(axis=(1, 3))
    thr = np.quantile(l1a, a_zero_frac)
    keep_a = np.repeat(np.repeat(l1a >= thr, 32, axis=0), 8, axis=1)[:M]
    A = A * keep_a
    nb = -(-N // 64)
    Bp = np.zeros((K, nb * 64), np.float32)
    Bp[:, :N] = B
    l1b = np.abs(Bp).reshape(nkb, 8, nb, 64).sum(axis=(1, 3))
    thr_b = np.quantile(l1b, 1.0 - b_keep_frac)
    keep_b = np.repeat(np.repeat(l1b >= thr_b, 8, axis=0), 64, axis=1)[:, :N]
    B = B * keep_b
    perm = rng.permutation(nkb)
    idx = (perm[:, None] * 8 + np.arange(8)[None, :]).ravel()
    return np.ascontiguousarray(A[:, idx], np.float32), np.ascontiguousarray(B[idx, :], np.float32)


def block_random(M, N, K, pa, pb, seed=0):
    """Whole 32 x 8 blocks of A and 8 x 32 blocks of B live with probability pa / pb (every pattern byte
    0x00 or 0xFF): what pruning at the pattern granularity produces."""
    rng = np.random.default_rng(seed)
    A = rng.standard_normal((M, K), dtype=np.float32)
    B = rng.standard_normal((K, N), dtype=np.float32)
    mb, nb, kb = -(-M // 32), -(-N // 32), -(-K // 8)
    la = (rng.random((mb, kb)) < pa).astype(np.float32)
    lb = (rng.random((nb, kb)) < pb).astype(np.float32)
    A *= np.repeat(np.repeat(la, 32, axis=0), 8, axis=1)[:M, :K]
    B *= np.repeat(np.repeat(lb, 32, axis=0), 8, axis=1)[:N, :K].T
    return A, B


def all_byte_values(M=256, N=256, seed=0):
    """A and B whose pattern arrays contain every byte value 0..255 (K = 256 * 8)."""
    K = 256 * 8
    rng = np.random.default_rng(seed)
    A = rng.standard_normal((M, K), dtype=np.float32)
    B = rng.standard_normal((K, N), dtype=np.float32)
    bits = np.array([[(v >> k) & 1 for k in range(8)] for v in range(256)], np.float32).ravel()
    permA = rng.permutation(256)
    la = np.stack([np.roll(bits.reshape(256, 8)[permA], r, axis=0).ravel() for r in range(-(-M // 32))])
    lb = np.stack([np.roll(bits.reshape(256, 8), 7 * r + 3, axis=0).ravel() for r in range(-(-N // 32))])
    A *= np.repeat(la, 32, axis=0)[:M]
    B *= np.repeat(lb, 32, axis=0)[:N].T
    return A, B
