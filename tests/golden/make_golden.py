"""Generate tests/golden/*.npz from the reference's own numpy oracles.

Runs only where the reference tree is present:

    python tests/golden/make_golden.py /path/to/reference

It imports python/examples/attention_training.py and python/examples/matmul.py
from that tree (their `triton_metal` shim needs a library exporting the tm_*
symbols: TRITON_METAL_CORE_LIB is pointed at libtmcuda.so, nothing is launched)
and stores the outputs of `numpy_attention`, `numpy_attention_backward` and
`a @ b` on seeded inputs, and of python/examples/sae_encode.py `reference` on that
example's own `synthetic` inputs.  Inputs are not stored: the tests regenerate them from
the seeds below.
"""

import os
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
ROOT = HERE.parents[1]

#: (name, heads, seq, dim, seed, input scale) - the example's own case
#: (attention_training.py:255-261), the pytest case (test_triton_roundtrip.py:97-132)
#: and two ragged Swift shapes (AttentionTests.swift:119-135).
ATTENTION_CASES = [
    ("h2_s96_d64_seed0", 2, 96, 64, 0, 0.5),
    ("h1_s48_d64_seed7", 1, 48, 64, 7, 0.5),
    ("h2_s127_d64_seed3", 2, 127, 64, 3, 1.0),
    ("h3_s33_d80_seed5", 3, 33, 80, 5, 1.0),
]


#: (rows, model width, features) - python/examples/sae_encode.py:120
SAE_CASES = [(8, 64, 128), (64, 512, 2048), (100, 300, 700)]


def attention_inputs(heads, seq, dim, seed, scale):
    rng = np.random.default_rng(seed)
    shape = (heads, seq, dim)
    return [rng.standard_normal(shape, dtype=np.float32) * np.float32(scale) for _ in range(4)]


def matmul_inputs(seed=0, n=256):
    rng = np.random.default_rng(seed)
    return (rng.standard_normal((n, n), dtype=np.float32),
            rng.standard_normal((n, n), dtype=np.float32))


def main(reference_root):
    os.environ.setdefault("TRITON_METAL_CORE_LIB",
                          str(ROOT / "triton-metal_b200" / "lib" / "libtmcuda.so"))
    sys.path.insert(0, str(Path(reference_root) / "python"))
    sys.path.insert(0, str(Path(reference_root) / "python" / "examples"))
    import attention_training as ref

    out = {}
    for name, heads, seq, dim, seed, scale in ATTENTION_CASES:
        q, k, v, target = attention_inputs(heads, seq, dim, seed, scale)
        sm = 1.0 / np.sqrt(dim)
        o, weights = ref.numpy_attention(q, k, v, sm)
        d_out = (o - target).astype(np.float32)
        dq, dk, dv = ref.numpy_attention_backward(q, k, v, weights, d_out, sm)
        for key, value in (("o", o), ("dq", dq), ("dk", dk), ("dv", dv)):
            out[f"{name}.{key}"] = np.asarray(value, dtype=np.float32)
    np.savez_compressed(HERE / "attention_reference.npz", **out)

    a, b = matmul_inputs()
    expected = a @ b          # python/examples/matmul.py:71
    np.savez_compressed(HERE / "matmul_reference.npz", rows=np.arange(0, 256, 16),
                        c_rows=expected[::16].copy(), checksum=np.float64(expected.astype(np.float64).sum()))
    # python/examples/sae_encode.py: `reference` on its own `synthetic` inputs, the three
    # shapes the example checks (:120) - sampled rows for the larger two
    import sae_encode as sae
    sae_out = {}
    for rows, model, features in SAE_CASES:
        x = sae.synthetic((rows, model), 1, 71)
        w = sae.synthetic((model, features), 7, 53)
        b = sae.synthetic((features,), 3, 29)
        want = sae.reference(x.astype(np.float64), w.astype(np.float64), b.astype(np.float64))
        key = f"m{rows}_d{model}_f{features}"
        sae_out[key + ".rows"] = np.arange(0, rows, max(1, rows // 8))
        sae_out[key + ".out"] = want[sae_out[key + ".rows"]].astype(np.float64)
        sae_out[key + ".x0"] = x.reshape(-1)[:16].copy()       # pins the input generator too
    np.savez_compressed(HERE / "sae_reference.npz", **sae_out)
    print("wrote", HERE / "attention_reference.npz", HERE / "matmul_reference.npz", HERE / "sae_reference.npz")


if __name__ == "__main__":
    import os
    if len(sys.argv) < 2 and not os.environ.get("TRITON_METAL_REFERENCE"):
        raise SystemExit("usage: make_golden.py <reference checkout>  (or set TRITON_METAL_REFERENCE)")
    main(sys.argv[1] if len(sys.argv) > 1 else os.environ["TRITON_METAL_REFERENCE"])
