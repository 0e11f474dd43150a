"""The one-dimensional kernels of the reference's own ABI tests, through the C ABI.

Cases follow Tests/TritonMetalCoreTests/CABITests.swift (vector add end to end :96-150,
unknown argument kind :152-173, f32 scalar arguments :263-308) and
python/tests/test_plugin_shape.py (vector add :184-215, softmax :220-259), plus the
masking rule of the Triton programs: nothing beyond min(n, grid * BLOCK) is touched."""

import ctypes
import json

import numpy as np
import pytest

import tmtest
from oracle import reference_math as ref
from triton_metal import _core, kernels
from triton_metal.buffer import MetalBuffer

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _gpu():
    tmtest.require_gpu()


def upload(array):
    return MetalBuffer.from_numpy(np.ascontiguousarray(array, dtype=np.float32))


def test_vector_add_round_trip():
    """n = 5000, a[i] = i/2, b[i] = i mod 13; bit-exact; every handle released."""
    n = 5000
    a = np.arange(n, dtype=np.float32) * np.float32(0.5)
    b = (np.arange(n) % 13).astype(np.float32)
    live = _core.live_handle_count()
    ir = kernels.elementwise_ir("add", 1024)
    meta = json.loads(_core.kernel_info(ir, 4))["kernels"][0]
    library = _core.compile_msl(_core.emit_msl(ir, 4))
    kernel = _core.load_kernel(library, meta["name"])
    assert _core.kernel_max_threads(kernel) >= meta["threads_per_threadgroup"]
    ba, bb = upload(a), upload(b)
    out = _core.alloc_buffer(4 * n)
    assert _core.buffer_length(out) == 4 * n
    block = meta["block_size"]
    _core.launch(kernel, ((n + block - 1) // block, 1, 1), meta["threads_per_threadgroup"],
                 [_core.ARG_BUFFER] * 3 + [_core.ARG_I32], [ba.tm_handle, bb.tm_handle, out, n])
    got = np.empty(n, dtype=np.float32)
    _core.buffer_read(out, 0, got.ctypes.data, got.nbytes)
    assert np.array_equal(got, ref.elementwise("add", a, b))
    ba.free(); bb.free(); _core.free_buffer(out)
    _core.release_kernel(kernel)
    _core.release_library(library)
    assert _core.live_handle_count() == live


@pytest.mark.parametrize("kind,block", [("copy", 256), ("add", 1024), ("mul", 128)])
@pytest.mark.parametrize("n", [1, 63, 1000, 4099, 1 << 20])
def test_elementwise_sizes_and_masking(kind, block, n):
    """Ragged sizes (tails of the 16-byte path), and a guard band behind element n."""
    rng = np.random.default_rng(n)
    a = rng.standard_normal(n + 8, dtype=np.float32)
    b = rng.standard_normal(n + 8, dtype=np.float32)
    sentinel = np.full(n + 8, -7.5, dtype=np.float32)
    kern = kernels.Elementwise(kind, block)
    ba, bb, bo = upload(a), upload(b), upload(sentinel)
    operands = (ba.tm_handle, bo.tm_handle) if kind == "copy" else (ba.tm_handle, bb.tm_handle, bo.tm_handle)
    kern(*operands, n=n)
    got = bo.numpy().copy()
    assert np.array_equal(got[:n], ref.elementwise(kind, a[:n], b[:n]))
    assert np.all(got[n:] == -7.5)
    kern.release()
    for buf in (ba, bb, bo):
        buf.free()


def test_programs_that_were_not_dispatched_leave_their_block_alone():
    n, block = 4096, 256
    a = np.arange(n, dtype=np.float32)
    kern = kernels.Elementwise("copy", block)
    ba, bo = upload(a), upload(np.zeros(n, dtype=np.float32))
    kern(ba.tm_handle, bo.tm_handle, n=n, programs=5)          # 16 programs would cover n
    got = bo.numpy()
    assert np.array_equal(got[:5 * block], a[:5 * block]) and not got[5 * block:].any()
    kern.release(); ba.free(); bo.free()


def test_float_scalars_travel_as_bit_patterns():
    """scale 2.5, bias -1.75 over 0..63: `x * scale + bias`, exactly."""
    n = 64
    x = np.arange(n, dtype=np.float32)
    kern = kernels.Elementwise("scale_bias", 64)
    bx, bo = upload(x), upload(np.full(n, np.nan, dtype=np.float32))
    kern(bx.tm_handle, bo.tm_handle, n=n, scale=2.5, bias=-1.75)
    assert np.array_equal(bo.numpy(), ref.elementwise("scale_bias", x, scale=2.5, bias=-1.75))
    # a product that is not exact in fp32: the kernel rounds it before adding, like the program
    x2 = np.linspace(0.1, 9.7, n, dtype=np.float32)
    bx.copy_from(x2.ctypes.data, x2.nbytes)
    kern(bx.tm_handle, bo.tm_handle, n=n, scale=1.1, bias=3.3)
    assert np.array_equal(bo.numpy(), ref.elementwise("scale_bias", x2, scale=1.1, bias=3.3))
    # a non-zero argument count with NULL arrays is a caller bug, not a crash
    lib = ctypes.CDLL(_core.library_path())
    lib.tm_launch.argtypes = [ctypes.c_int64] * 5 + [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int32]
    assert lib.tm_launch(kern.handle, 1, 1, 1, 128, None, None, 5) == -1
    assert "NULL argument arrays" in _core.last_error()
    kern.release(); bx.free(); bo.free()


def test_unknown_argument_kind_is_rejected():
    kern = kernels.Elementwise("copy", 256)
    with pytest.raises(RuntimeError, match="unknown launch argument kind 7"):
        _core.launch(kern.handle, (1, 1, 1), 32, [7], [0])
    kern.release()


def test_buffers_too_short_for_the_launch_are_refused():
    kern = kernels.Elementwise("add", 1024)
    ba, bb, bo = (upload(np.zeros(100, dtype=np.float32)) for _ in range(3))
    with pytest.raises(RuntimeError, match="beyond its 400-byte buffer"):
        kern(ba.tm_handle, bb.tm_handle, bo.tm_handle, n=101)
    kern.release()
    for buf in (ba, bb, bo):
        buf.free()


def test_softmax_round_trip():
    """12 rows of 100 columns in a BLOCK of 128; rel 1e-5, abs 1e-7."""
    rows, n_cols = 12, 100
    data = (((np.arange(rows * n_cols) * 17) % 53) * 0.4 - 10).astype(np.float32)
    live = _core.live_handle_count()
    kern = kernels.Softmax(128)
    bx, bo = upload(data), upload(np.zeros(rows * n_cols, dtype=np.float32))
    kern(bx.tm_handle, bo.tm_handle, rows, n_cols)
    got = bo.numpy().reshape(rows, n_cols)
    want = ref.softmax_rows(data.reshape(rows, n_cols))
    assert np.all(np.abs(got - want) <= 1e-5 * np.abs(want) + 1e-7)
    kern.release(); bx.free(); bo.free()
    assert _core.live_handle_count() == live


def test_softmax_strides_block_limit_and_many_rows():
    """Padded rows; columns beyond BLOCK are never read or written; more rows than CTAs."""
    rows, n_cols, stride = 5000, 200, 208
    rng = np.random.default_rng(3)
    x = rng.standard_normal((rows, stride), dtype=np.float32) * 4
    kern = kernels.Softmax(128)
    bx, bo = upload(x), upload(np.full((rows, stride), -2.0, dtype=np.float32))
    kern(bx.tm_handle, bo.tm_handle, rows, n_cols, stride, stride)
    got = bo.numpy().reshape(rows, stride)
    want = ref.softmax_rows(x[:, :128])
    assert np.all(np.abs(got[:, :128] - want) <= 1e-5 * np.abs(want) + 1e-7)
    assert np.all(got[:, 128:] == -2.0)
    kern.release(); bx.free(); bo.free()
