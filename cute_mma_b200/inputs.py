"""Seeded synthetic operands for the OFT / GEMM path (host side, numpy).

The reference's drivers draw A, B from per-thread mt19937 streams seeded by wall-clock time
(cute_oft_pc.cu:195-236) and the GEMM driver from unseeded rand() (gemm_sm80_tc.cu:499-502), so its
inputs are not reproducible.  This module pins one generator (numpy PCG64 via default_rng(seed)) and
supplies the block builders the benchmark configurations name.

Storage convention (cpu_oft.hpp:52-64,101-108): the block stored at rows g*b+q, columns kb*b+p holds
R_math[p][q], i.e. the stored block is the transpose of the mathematical rotation in
Y = sum_kb (X_kb . R_math) . W_kb.  pack_r() applies that transpose.
"""
from __future__ import annotations

import numpy as np


def rng(seed: int) -> np.random.Generator:
    return np.random.default_rng(seed)


def uniform_pm1(shape, seed: int, dtype=np.float16) -> np.ndarray:
    """U(-1, 1)."""
    return rng(seed).uniform(-1.0, 1.0, size=shape).astype(dtype)


def uniform_01(shape, seed: int, dtype=np.float16) -> np.ndarray:
    """U[0, 1): the positive inputs the reference uses so that relative error is stable."""
    return rng(seed).uniform(0.0, 1.0, size=shape).astype(dtype)


def zero_one(shape, seed: int, dtype=np.float16) -> np.ndarray:
    """Entries in {0, 1} (--01init, cute_oft_pc.cu:202-216): small-integer sums, exact in fp16."""
    return rng(seed).integers(0, 2, size=shape).astype(dtype)


def normal(shape, seed: int, sigma: float = 1.0, dtype=np.float16) -> np.ndarray:
    return (rng(seed).standard_normal(size=shape) * sigma).astype(dtype)


# ---- orthogonal block builders: each returns R_math blocks, float64, shape [n_groups, n_blocks, b, b]


def blocks_qr(n_groups: int, n_blocks: int, b: int, seed: int) -> np.ndarray:
    """Q factor of a seeded N(0,1) matrix per block."""
    g = rng(seed)
    out = np.empty((n_groups, n_blocks, b, b))
    for i in range(n_groups):
        for j in range(n_blocks):
            q, r = np.linalg.qr(g.standard_normal((b, b)))
            out[i, j] = q * np.sign(np.diag(r))  # fix the sign ambiguity so the result is unique
    return out


def blocks_cayley(n_groups: int, n_blocks: int, b: int, seed: int, sigma: float = 0.01) -> np.ndarray:
    """Cayley transform (I - S)(I + S)^-1 of a seeded skew-symmetric S with entries ~ N(0, sigma)."""
    g = rng(seed)
    eye = np.eye(b)
    out = np.empty((n_groups, n_blocks, b, b))
    for i in range(n_groups):
        for j in range(n_blocks):
            a = g.standard_normal((b, b)) * sigma
            s = np.triu(a, 1)
            s = s - s.T
            out[i, j] = (eye - s) @ np.linalg.inv(eye + s)
    return out


def blocks_permutation(n_groups: int, n_blocks: int, b: int, seed: int) -> np.ndarray:
    """Random permutation matrices (cute_oft_pc.cu:222-235): exact in fp16 and not symmetric, so a
    transposed-R bug changes the result while X.R itself stays exact."""
    g = rng(seed)
    out = np.zeros((n_groups, n_blocks, b, b))
    for i in range(n_groups):
        for j in range(n_blocks):
            perm = g.permutation(b)
            out[i, j, np.arange(b), perm] = 1.0
    return out


def blocks_structured(n_groups: int, n_blocks: int, b: int) -> np.ndarray:
    """Known-answer block in the spirit of playgrounds/bd_construct.cu:117-123:
    R_math = I + E with E[0][0] = 1 and E[0][q] = 1 for q >= 1, so (x . R_math)[q] = x[q] + x[0]
    for q >= 1 and 2 x[0] for q = 0."""
    blk = np.eye(b)
    blk[0, :] += 1.0
    return np.broadcast_to(blk, (n_groups, n_blocks, b, b)).copy()


def pack_r(blocks: np.ndarray, dtype=np.float16) -> np.ndarray:
    """[G, KB, b, b] R_math blocks -> stored R [G*b, KB*b] with every block transposed."""
    G, KB, b, _ = blocks.shape
    # stored[g*b+q, kb*b+p] = blocks[g, kb, p, q]
    return np.ascontiguousarray(blocks.transpose(0, 3, 1, 2).reshape(G * b, KB * b)).astype(dtype)


def unpack_r(stored: np.ndarray, b: int) -> np.ndarray:
    """Inverse of pack_r (as float64)."""
    Gb, K = stored.shape
    return stored.astype(np.float64).reshape(Gb // b, b, K // b, b).transpose(0, 2, 3, 1).copy()


def oft_flops(m: int, n: int, k: int, b: int, n_groups: int = 1) -> float:
    """Algorithmic FLOPs credited to the fused product, AR_W counting (cute_oft_pc.cu:362-367)."""
    return 2.0 * m * n * k + 2.0 * n_groups * m * k * b


def gemm_flops(m: int, n: int, k: int) -> float:
    return 2.0 * m * n * k
