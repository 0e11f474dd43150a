"""Seeded synthetic inputs for every benchmark / parity configuration.

TEST INFRASTRUCTURE ONLY - see oracle/__init__.py.  The generators stand in for
the reference's tutorial shapes; no public dataset is involved.
"""

import numpy as np


def gemm_uniform(M, N, K, seed=0):
    """fp32 A[M,K], B[K,N] i.i.d. uniform[-1,1)."""
    rng = np.random.default_rng(seed)
    a = rng.uniform(-1.0, 1.0, size=(M, K)).astype(np.float32)
    b = rng.uniform(-1.0, 1.0, size=(K, N)).astype(np.float32)
    return a, b


def gemm_normal(M, N, K, seed=0):
    """A, B ~ N(0,1)/sqrt(K) in float32 (round to the storage type afterwards)."""
    rng = np.random.default_rng(seed)
    a = (rng.standard_normal((M, K), dtype=np.float32) / np.float32(np.sqrt(K)))
    b = (rng.standard_normal((K, N), dtype=np.float32) / np.float32(np.sqrt(K)))
    return a, b


def attention_normal(bh, seq, head_dim, seed=0, count=4, scale=1.0):
    """`count` tensors [bh, seq, head_dim] ~ N(0, scale^2) (Q, K, V, dO)."""
    rng = np.random.default_rng(seed)
    return [rng.standard_normal((bh, seq, head_dim), dtype=np.float32) * np.float32(scale)
            for _ in range(count)]


def closed_form_matrix(rows, cols, modulus, scale=0.01, shift=0.5):
    """The reference benchmarks' closed-form fill `(i % modulus) * scale - shift`
    (Sources/TritonMetalBench/GEMMBenchmark.swift:386-387)."""
    i = np.arange(rows * cols, dtype=np.int64)
    return ((i % modulus).astype(np.float32) * np.float32(scale) - np.float32(shift)).reshape(rows, cols)


def closed_form_tensor(shape, seed):
    """`(i % seed) / seed - 0.5`
    (Sources/TritonMetalBench/AttentionBackwardBenchmark.swift:489-491)."""
    n = int(np.prod(shape))
    i = np.arange(n, dtype=np.int64)
    return ((i % seed).astype(np.float32) / np.float32(seed) - np.float32(0.5)).reshape(shape)


def sae_synthetic(shape, offset, modulus):
    """Deterministic values in [-0.5, 0.5): ((i + offset) * 13 mod modulus) / modulus - 0.5
    (python/examples/sae_encode.py:61-65)."""
    count = int(np.prod(shape))
    i = np.arange(count, dtype=np.int64)
    return (((i + offset) * 13 % modulus) / modulus - 0.5).astype(np.float32).reshape(shape)


def sae_inputs(rows, model, features):
    """x, W_enc, b_enc of the example's checks (sae_encode.py:121-123)."""
    return (sae_synthetic((rows, model), 1, 71), sae_synthetic((model, features), 7, 53),
            sae_synthetic((features,), 3, 29))
