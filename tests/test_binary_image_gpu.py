"""A binary image behind tm_load_metallib: the caller's own CUDA kernels through the reference's
library / kernel / launch calls (Compiler.swift:250-263 loads a precompiled metallib the same
way; Runtime.swift:182-243 binds argument i at index i).  The image is built here with nvcc from
a few lines of CUDA; the expectations are numpy expressions."""

import os
import shutil
import subprocess

import numpy as np
import pytest

import tmtest
from triton_metal import _core

pytestmark = pytest.mark.gpu

SOURCE = r"""
extern "C" __global__ void saxpy_kernel(const float* x, const float* y, float* out, float a, int n) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = a * x[i] + y[i];
}
extern "C" __global__ void iota64_kernel(long long* out, long long first, int n) {
  int i = (blockIdx.y * gridDim.x + blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) out[i] = first + i;
}
"""


@pytest.fixture(scope="module")
def image(tmp_path_factory):
    tmtest.require_gpu()
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        pytest.skip("no nvcc on this machine to build the image")
    d = tmp_path_factory.mktemp("image")
    (d / "k.cu").write_text(SOURCE)
    subprocess.run([nvcc, "-cubin", "-fmad=false", "-gencode", "arch=compute_100a,code=sm_100a", "-o", str(d / "k.cubin"),
                    str(d / "k.cu")], check=True)
    return (d / "k.cubin").read_bytes()


def test_kernels_of_a_cubin_run_through_the_launch_call(image):
    live = _core.live_handle_count()
    library = _core.load_metallib(image)
    saxpy = _core.load_kernel(library, "saxpy_kernel")
    iota = _core.load_kernel(library, "iota64_kernel")
    assert 1 <= _core.kernel_max_threads(saxpy) <= 1024
    n = 100003
    rng = np.random.default_rng(3)
    x, y = rng.standard_normal(n).astype(np.float32), rng.standard_normal(n).astype(np.float32)
    bx, by, bo = (_core.alloc_buffer(4 * n) for _ in range(3))
    b64 = _core.alloc_buffer(8 * n)
    try:
        _core.buffer_write(bx, 0, x.ctypes.data, x.nbytes)
        _core.buffer_write(by, 0, y.ctypes.data, y.nbytes)
        a = np.float32(1.75)
        _core.launch(saxpy, ((n + 255) // 256, 1, 1), 256,
                     [_core.ARG_BUFFER] * 3 + [_core.ARG_F32, _core.ARG_I32], [bx, by, bo, _core.float_bits(float(a)), n])
        got = np.empty(n, dtype=np.float32)
        _core.buffer_read(bo, 0, got.ctypes.data, got.nbytes)
        assert np.array_equal(got, a * x + y)
        # a two-dimensional grid and a 64-bit scalar
        first = (1 << 40) + 5
        _core.launch(iota, (7, (n + 7 * 128 - 1) // (7 * 128), 1), 128,
                     [_core.ARG_BUFFER, _core.ARG_I64, _core.ARG_I32], [b64, first, n])
        got64 = np.empty(n, dtype=np.int64)
        _core.buffer_read(b64, 0, got64.ctypes.data, got64.nbytes)
        assert np.array_equal(got64, first + np.arange(n, dtype=np.int64))
    finally:
        for h in (bx, by, bo, b64):
            _core.free_buffer(h)
        _core.release_kernel(saxpy)
        _core.release_kernel(iota)
        _core.release_library(library)
    assert _core.live_handle_count() == live


def test_a_kernel_outlives_the_release_of_its_library(image):
    library = _core.load_metallib(image)
    iota = _core.load_kernel(library, "iota64_kernel")
    _core.release_library(library)
    out = _core.alloc_buffer(8 * 64)
    try:
        _core.launch(iota, (1, 1, 1), 64, [_core.ARG_BUFFER, _core.ARG_I64, _core.ARG_I32], [out, -3, 64])
        got = np.empty(64, dtype=np.int64)
        _core.buffer_read(out, 0, got.ctypes.data, got.nbytes)
        assert np.array_equal(got, np.arange(64) - 3)
    finally:
        _core.free_buffer(out)
        _core.release_kernel(iota)


def test_mismatched_launches_are_messages_not_faults(image):
    library = _core.load_metallib(image)
    saxpy = _core.load_kernel(library, "saxpy_kernel")
    buf = _core.alloc_buffer(1024)
    try:
        with pytest.raises(RuntimeError, match="not found in library \\(available: iota64_kernel, saxpy_kernel\\)"):
            _core.load_kernel(library, "missing_kernel")
        with pytest.raises(RuntimeError, match="takes 5 arguments, got 4"):
            _core.launch(saxpy, (1, 1, 1), 32, [_core.ARG_BUFFER] * 3 + [_core.ARG_I32], [buf, buf, buf, 8])
        with pytest.raises(RuntimeError, match="argument 3 of kernel 'saxpy_kernel' is 4 bytes wide, the launch passes 8"):
            _core.launch(saxpy, (1, 1, 1), 32, [_core.ARG_BUFFER] * 3 + [_core.ARG_I64, _core.ARG_I32],
                         [buf, buf, buf, 1, 8])
        with pytest.raises(RuntimeError, match="unknown launch argument kind 9 at position 4"):
            _core.launch(saxpy, (1, 1, 1), 32, [_core.ARG_BUFFER] * 3 + [_core.ARG_F32, 9], [buf, buf, buf, _core.float_bits(1.0), 8])
        with pytest.raises(RuntimeError, match="exceeds the pipeline maximum"):
            _core.launch(saxpy, (1, 1, 1), 2048, [_core.ARG_BUFFER] * 3 + [_core.ARG_F32, _core.ARG_I32],
                         [buf, buf, buf, _core.float_bits(1.0), 8])
        with pytest.raises(RuntimeError, match="grid must be positive"):
            _core.launch(saxpy, (0, 1, 1), 32, [_core.ARG_BUFFER] * 3 + [_core.ARG_F32, _core.ARG_I32],
                         [buf, buf, buf, _core.float_bits(1.0), 8])
        # the context is still fine
        _core.launch(saxpy, (1, 1, 1), 32, [_core.ARG_BUFFER] * 3 + [_core.ARG_F32, _core.ARG_I32],
                     [buf, buf, buf, _core.float_bits(1.0), 8])
    finally:
        _core.free_buffer(buf)
        _core.release_kernel(saxpy)
        _core.release_library(library)


def test_an_image_that_is_not_a_binary_is_refused():
    tmtest.require_gpu()
    with pytest.raises(RuntimeError, match="could not load metallib"):
        _core.load_metallib(b"\x7fELF" + bytes(200))
