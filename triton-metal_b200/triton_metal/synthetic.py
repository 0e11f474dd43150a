"""Seeded synthetic inputs in storage format (bf16 as uint16 words) for the
benchmark drivers.  The distributions are the ones the benchmark configurations
name: GEMM operands N(0,1)/sqrt(K), attention tensors N(0,1)."""

import numpy as np


def to_bf16_bits(x):
    """float32 -> bf16 bit patterns, round to nearest even."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    rounded = u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))
    return (rounded >> np.uint32(16)).astype(np.uint16)


def from_bf16_bits(bits):
    return (np.ascontiguousarray(bits, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


def gemm_inputs_bf16(M, N, K, seed, row0=0, rows=None):
    """Rows [row0, row0+rows) of A[M,K] and all of B[K,N].  Every rank derives
    the same B from `seed` and its own rows of A from (seed, row block)."""
    rows = M if rows is None else rows
    scale = np.float32(1.0 / np.sqrt(K))
    b = np.random.default_rng([seed, 1]).standard_normal((K, N), dtype=np.float32) * scale
    a = np.random.default_rng([seed, 2, row0]).standard_normal((rows, K), dtype=np.float32) * scale
    return to_bf16_bits(a), to_bf16_bits(b)


def attention_inputs_bf16(bh, seq, head_dim, seed, count):
    rng = np.random.default_rng([seed, 3])
    return [to_bf16_bits(rng.standard_normal((max(bh, 1), seq, head_dim), dtype=np.float32))[:bh]
            if bh else np.zeros((0, seq, head_dim), dtype=np.uint16) for _ in range(count)]
