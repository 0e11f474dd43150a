"""sae_encode_kernel - relu(x @ W_enc + b_enc) fused into the matmul - through the C ABI.

Shapes, inputs and the error measure follow python/examples/sae_encode.py:120-131 and
Tests/TritonMetalMLXTests/SAEEncoderTests.swift:25-45 (max |kernel - float64 reference| over
max(|reference|, 1) below 2e-6); the large shapes run on the tensor cores (3xTF32) and are held
to the fp32 parity bound of the matmul, 1e-5."""

from pathlib import Path

import numpy as np
import pytest

import tmtest
from oracle import inputs, reference_math as ref
from triton_metal import cuda, kernels
from triton_metal.buffer import MetalBuffer

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden"


@pytest.fixture(autouse=True)
def _gpu():
    tmtest.require_gpu()


def encode(x, w, b, block=(64, 64, 16), path=0, programs=None, out_init=None):
    rows, model = x.shape
    features = w.shape[1]
    kern = kernels.SaeEncode(block)
    kern.set_path(path)
    bufs = [MetalBuffer.from_numpy(np.ascontiguousarray(t, dtype=np.float32)) for t in (x, w, b)]
    out = MetalBuffer.from_numpy(np.zeros((rows, features), dtype=np.float32) if out_init is None else out_init)
    grid, kinds, values = kern.arguments(*(t.tm_handle for t in bufs), out.tm_handle, rows, model, features)
    if programs is not None:
        grid = programs
    kern.launch(grid, kinds, values)
    got = out.numpy().reshape(rows, features).copy()
    used = kern.last_path()
    kern.release()
    for t in bufs + [out]:
        t.free()
    return got, used


def scaled_error(got, want):
    return float(np.max(np.abs(got - want))) / max(float(np.max(np.abs(want))), 1.0)


@pytest.mark.parametrize("rows,model,features", [(8, 64, 128), (64, 512, 2048), (100, 300, 700)])
def test_example_shapes(rows, model, features):
    x, w, b = inputs.sae_inputs(rows, model, features)
    want = ref.sae_encode(x.astype(np.float64), w.astype(np.float64), b.astype(np.float64))
    golden = np.load(GOLDEN / "sae_reference.npz")
    key = f"m{rows}_d{model}_f{features}"
    for block in ((64, 64, 16), (32, 64, 32)):
        got, _ = encode(x, w, b, block)
        assert scaled_error(got, want) < 2e-6
        assert scaled_error(got[golden[key + ".rows"]], golden[key + ".out"]) < 2e-6
        assert np.all(got >= 0)


def test_negative_preactivations_are_exact_zeros():
    rng = np.random.default_rng(0)
    x = np.abs(rng.standard_normal((70, 96), dtype=np.float32))
    w = -np.abs(rng.standard_normal((96, 130), dtype=np.float32))
    b = np.full(130, -0.5, dtype=np.float32)
    got, _ = encode(x, w, b)
    assert not got.any()
    b[::2] = 1e6                                   # every other feature is pushed positive
    got, _ = encode(x, w, b)
    assert np.all(got[:, ::2] > 0) and not got[:, 1::2].any()


def test_tiles_that_were_not_dispatched_stay_untouched():
    x, w, b = inputs.sae_inputs(128, 64, 256)
    sentinel = np.full((128, 256), -3.0, dtype=np.float32)
    got, _ = encode(x, w, b, programs=(1, 2, 1), out_init=sentinel)      # 64 rows x 128 features
    want = ref.sae_encode(x.astype(np.float64), w.astype(np.float64), b.astype(np.float64))
    assert scaled_error(got[:64, :128], want[:64, :128]) < 2e-6
    assert np.all(got[64:] == -3.0) and np.all(got[:, 128:] == -3.0)


@pytest.mark.parametrize("rows,model,features", [(1024, 512, 4096), (4096, 1024, 8192), (1000, 520, 4100)])
def test_large_shapes_on_the_tensor_cores(rows, model, features):
    """An SAE over a residual stream: features >> model width.  The 3xTF32 path with the fused
    epilogue against the generic fp32 kernel and the float64 reference on sampled rows."""
    rng = np.random.default_rng(rows)
    x = rng.standard_normal((rows, model), dtype=np.float32)
    w = rng.standard_normal((model, features), dtype=np.float32) / np.float32(np.sqrt(model))
    b = rng.standard_normal(features, dtype=np.float32) * np.float32(0.5)
    got, used = encode(x, w, b, (128, 256, 32))
    assert used == cuda.PATH_TCGEN05
    picked = np.arange(0, rows, max(1, rows // 64))
    want = ref.sae_encode(x[picked].astype(np.float64), w.astype(np.float64), b.astype(np.float64))
    assert ref.relative_error(got[picked], want) <= 1e-5
    assert scaled_error(got[picked], want) <= 1e-5
    assert np.all(got >= 0)
    simt, used = encode(x, w, b, (128, 256, 32), path=cuda.PATH_SIMT)
    assert used == cuda.PATH_SIMT
    assert ref.relative_error(got, simt) <= 1e-5
    assert np.mean((got == 0) == (simt == 0)) > 0.9999      # the ReLU cuts at the same places
