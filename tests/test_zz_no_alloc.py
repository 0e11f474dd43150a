"""The allocation-free fp32 matmul entry point (tmx_matmul_f32_static).

Some hosts cannot let a library allocate device memory behind their back: they have
already carved all of HBM into their own pool, or they are past the point in their life
cycle where allocation is allowed.  For them the fp32 matmul - whose 3xTF32 operand split
needs scratch - exists in a second form whose scratch is a fixed array inside the library.
This file checks that form against the ordinary one (tm_launch), through the C ABI, on
two calls in a row that share the array, and checks the documented size limit.

Collected last on purpose: a failure here must not hide the results of any other test.
"""

import numpy as np
import pytest

import tmtest
from oracle import inputs, reference_math as ref
from triton_metal import cuda, kernels

pytestmark = pytest.mark.gpu


def _both_ways(M, N, K, seed):
    a, b = inputs.gemm_uniform(M, N, K, seed=seed)
    ab, bb = tmtest.upload(a, "f32"), tmtest.upload(b, "f32")
    c_launch, c_static = tmtest.empty((M, N), "f32"), tmtest.empty((M, N), "f32")
    mm = kernels.Matmul("f32", (128, 128, 32))
    try:
        mm.set_path(cuda.PATH_TCGEN05)
        mm(ab.tm_handle, bb.tm_handle, c_launch.tm_handle, M, N, K)
        cuda.matmul_f32_static(ab.tm_handle, bb.tm_handle, c_static.tm_handle, M, N, K)
        return tmtest.fetch(c_launch), tmtest.fetch(c_static), ref.matmul(a, b)
    finally:
        mm.release()
        for buf in (ab, bb, c_launch, c_static):
            buf.free()


def test_static_scratch_matmul_matches_tm_launch_twice_in_a_row():
    tmtest.require_gpu()
    # the second problem is smaller in every extent: anything the first call left in the
    # shared array beyond it must not leak into the result
    for M, N, K in ((512, 384, 600), (256, 128, 136)):
        got_launch, got_static, want = _both_ways(M, N, K, seed=M + K)
        assert ref.relative_error(got_static, got_launch) <= 1e-5
        assert ref.relative_error(got_static, want) <= 1e-5


def test_static_scratch_matmul_takes_strided_operands_and_allocates_nothing():
    """A transposed A, a padded B and a padded C (stride_am = 1, row strides wider than the rows)
    through the fixed-array entry point; and, once the first call has loaded the module, a
    call leaves the amount of free device memory exactly as it found it."""
    tmtest.require_gpu()
    M, N, K = 256, 192, 320
    a, b = inputs.gemm_normal(M, N, K, seed=4)
    a_t = np.ascontiguousarray(a.T)
    b_pad = np.zeros((K, N + 5), dtype=np.float32)
    b_pad[:, :N] = b
    ab, bb = tmtest.upload(a_t, "f32"), tmtest.upload(b_pad, "f32")
    cb = tmtest.empty((M, N + 3), "f32")
    try:
        cuda.matmul_f32_static_prepare()
        strides = (1, M, N + 5, 1, N + 3, 1)
        tmtest.put(cb, np.full((M, N + 3), -9.0, dtype=np.float32))
        cuda.matmul_f32_static(ab.tm_handle, bb.tm_handle, cb.tm_handle, M, N, K, strides)
        free_before, _ = cuda.device_memory()
        tmtest.put(cb, np.full((M, N + 3), -9.0, dtype=np.float32))
        cuda.matmul_f32_static(ab.tm_handle, bb.tm_handle, cb.tm_handle, M, N, K, strides)
        free_after, _ = cuda.device_memory()
        c = tmtest.fetch(cb)
        assert free_after == free_before
        assert ref.relative_error(c[:, :N], ref.matmul(a, b)) <= 1e-5
        assert np.all(c[:, N:] == -9.0)
    finally:
        for buf in (ab, bb, cb):
            buf.free()


def test_static_scratch_matmul_refuses_what_does_not_fit(core):
    tmtest.require_gpu()
    capacity = cuda.matmul_f32_static_capacity()
    assert capacity == 8 << 20
    M, N, K = 2048, 2048, 2048                       # needs 8*(M+N)*K = 64 MiB of scratch
    assert 8 * (M + N) * K > capacity
    big = tmtest.empty((M, K), "f32")
    try:
        with pytest.raises(RuntimeError, match="more than the 8388608-byte fixed array"):
            cuda.matmul_f32_static(big.tm_handle, big.tm_handle, big.tm_handle, M, N, K)
        with pytest.raises(RuntimeError, match="at least 128 x 64 x 32"):
            cuda.matmul_f32_static(big.tm_handle, big.tm_handle, big.tm_handle, 64, 64, 64)
        with pytest.raises(RuntimeError, match="beyond its"):
            cuda.matmul_f32_static(big.tm_handle, big.tm_handle, big.tm_handle, 4096, 128, 2048)
        # extents and strides whose product does not fit 64 bits are refused, not wrapped
        with pytest.raises(RuntimeError, match="beyond its|above 2\\^31"):
            cuda.matmul_f32_static(big.tm_handle, big.tm_handle, big.tm_handle, 1 << 31, 128, 64,
                                   (1 << 33, 1, 128, 1, 128, 1))
        with pytest.raises(RuntimeError, match="beyond its"):
            cuda.matmul_f32_static(big.tm_handle, big.tm_handle, big.tm_handle, 1 << 20, 128, 64,
                                   (1 << 44, 1, 128, 1, 128, 1))
    finally:
        big.free()
