"""matmul_kernel parity through the C ABI, against the numpy oracle.

Shapes and tolerances follow Tests/TritonMetalCoreTests/DotTests.swift (ragged
shapes tol 1e-5 :369-396, strides :403-461, f16 :466-506, bf16 from already
rounded inputs :514-554, guard bands :609-646) and the benchmark configurations
(fp32 256^3 uniform[-1,1); bf16 N(0,1)/sqrt(K) squares and the skinny shape)."""

import numpy as np
import pytest

import tmtest
from oracle import inputs, reference_math as ref
from triton_metal import cuda

pytestmark = pytest.mark.gpu

TOL = {"f32": 1e-5, "f16": 2e-2, "bf16": 2e-2}


@pytest.fixture(autouse=True)
def _gpu():
    tmtest.require_gpu()


def test_fp32_256_cubed_uniform():
    a, b = inputs.gemm_uniform(256, 256, 256, seed=0)
    for block in ((128, 64, 32), (64, 64, 32), (64, 64, 64), (32, 32, 32)):
        c, _ = tmtest.run_matmul(a, b, "f32", block)
        assert ref.relative_error(c, ref.matmul(a, b)) <= 1e-5
        assert float(np.max(np.abs(c - ref.matmul(a, b)))) < 1e-3     # matmul.py:78


@pytest.mark.parametrize("shape", [(64, 64, 64), (129, 257, 65), (33, 17, 129), (1, 1, 1),
                                   (128, 96, 40), (200, 120, 72)])
@pytest.mark.parametrize("element", ["f32", "f16", "bf16"])
def test_ragged_shapes(shape, element):
    M, N, K = shape
    a, b = inputs.gemm_normal(M, N, K, seed=M + N + K)
    a, b = ref.round_to(a, element), ref.round_to(b, element)
    c, _ = tmtest.run_matmul(a, b, element, (64, 64, 16))
    assert ref.relative_error(c, ref.matmul(a, b)) <= TOL[element]


def test_non_unit_and_padded_strides():
    """A read through a transposed view, B with padded rows, C with padded rows."""
    M, N, K = 96, 80, 72
    a, b = inputs.gemm_normal(M, N, K, seed=5)
    a_t = np.ascontiguousarray(a.T)                     # stored [K, M]: stride_am=1, stride_ak=M
    b_pad = np.zeros((K, N + 24), dtype=np.float32)
    b_pad[:, :N] = b
    strides = (1, M, N + 24, 1, N + 8, 1)
    ab, bb = tmtest.upload(a_t, "f32"), tmtest.upload(b_pad, "f32")
    cb = tmtest.empty((M, N + 8), "f32")
    from triton_metal import kernels
    mm = kernels.Matmul("f32", (32, 32, 16))
    try:
        mm(ab.tm_handle, bb.tm_handle, cb.tm_handle, M, N, K, strides)
        c = tmtest.fetch(cb)
        assert ref.relative_error(c[:, :N], ref.matmul(a, b)) <= 1e-5
        assert np.all(c[:, N:] == 0)                    # padding columns untouched
    finally:
        mm.release()
        for buf in (ab, bb, cb):
            buf.free()


@pytest.mark.parametrize("element", ["f32", "bf16"])
def test_masked_stores_never_touch_the_guard_band(element):
    """C lives inside a larger buffer filled with a sentinel."""
    M, N, K = 129, 136, 65
    a, b = inputs.gemm_normal(M, N, K, seed=9)
    a, b = ref.round_to(a, element), ref.round_to(b, element)
    rows, cols = M + 7, N + 8
    c, _ = tmtest.run_matmul(a, b, element, (64, 64, 16), strides=(K, 1, N, 1, cols, 1),
                             c_shape=(rows, cols), c_fill=-7.0)
    assert ref.relative_error(c[:M, :N], ref.matmul(a, b)) <= TOL[element]
    assert np.all(c[M:, :] == -7.0) and np.all(c[:, N:] == -7.0)


def test_programs_outside_the_grid_are_not_run():
    """A grid smaller than cdiv(M,BM) x cdiv(N,BN) leaves the other tiles alone."""
    a, b = inputs.gemm_normal(128, 128, 64, seed=2)
    c, _ = tmtest.run_matmul(a, b, "f32", (64, 64, 16), c_fill=3.0, grid=(1, 2, 1))
    want = ref.matmul(a, b)
    assert ref.relative_error(c[:64], want[:64]) <= 1e-5
    assert np.all(c[64:] == 3.0)


@pytest.mark.parametrize("element", ["bf16", "f16"])
@pytest.mark.parametrize("n", [1024, 2048])
def test_square_16bit_takes_the_tensor_core_path(element, n):
    a, b = inputs.gemm_normal(n, n, n, seed=n)
    a, b = ref.round_to(a, element), ref.round_to(b, element)
    c, path = tmtest.run_matmul(a, b, element)
    assert path == cuda.PATH_TCGEN05
    assert ref.relative_error(c, ref.matmul(a, b)) <= TOL[element]


@pytest.mark.parametrize("shape", [(128, 64, 64), (256, 264, 72), (384, 520, 200), (1000, 776, 136),
                                   (130, 72, 64)])
def test_tensor_core_path_ragged_edges(shape):
    M, N, K = shape
    a, b = inputs.gemm_normal(M, N, K, seed=M ^ N ^ K)
    a, b = ref.round_to(a, "bf16"), ref.round_to(b, "bf16")
    rows, cols = M + 3, N + 8
    c, path = tmtest.run_matmul(a, b, "bf16", path=cuda.PATH_TCGEN05,
                                strides=(K, 1, N, 1, cols, 1), c_shape=(rows, cols), c_fill=-5.0)
    assert path == cuda.PATH_TCGEN05
    assert ref.relative_error(c[:M, :N], ref.matmul(a, b)) <= 2e-2
    assert np.all(c[M:, :] == -5.0) and np.all(c[:, N:] == -5.0)


def test_both_paths_agree_on_bf16():
    a, b = inputs.gemm_normal(512, 512, 512, seed=3)
    a, b = ref.round_to(a, "bf16"), ref.round_to(b, "bf16")
    c_tc, p1 = tmtest.run_matmul(a, b, "bf16", path=cuda.PATH_TCGEN05)
    c_simt, p2 = tmtest.run_matmul(a, b, "bf16", path=cuda.PATH_SIMT)
    assert (p1, p2) == (cuda.PATH_TCGEN05, cuda.PATH_SIMT)
    # both round an fp32 accumulation once: they may differ by one bf16 ulp at most
    assert ref.relative_error(c_tc, c_simt) <= 2 ** -7


def test_large_bf16_against_sampled_oracle_rows():
    """4096^3: the oracle checks sampled row blocks; linearity covers the rest."""
    n = 4096
    a, b = inputs.gemm_normal(n, n, n, seed=7)
    a, b = ref.round_to(a, "bf16"), ref.round_to(b, "bf16")
    c, path = tmtest.run_matmul(a, b, "bf16")
    assert path == cuda.PATH_TCGEN05
    rows = np.r_[0:64, 2000:2064, n - 64:n]
    assert ref.relative_error(c[rows], ref.matmul(a[rows], b)) <= 2e-2
    # checksum of checksums: column sums of C equal (column sums of A) @ B
    want = a.astype(np.float64).sum(axis=0) @ b.astype(np.float64)
    got = c.astype(np.float64).sum(axis=0)
    assert np.max(np.abs(got - want)) / np.max(np.abs(want)) < 2e-2


def test_skinny_bf16_shape_sampled():
    M, N, K = 16384, 4096, 14336
    rng = np.random.default_rng(1)
    a = ref.round_to(rng.standard_normal((M, K), dtype=np.float32) / np.float32(np.sqrt(K)), "bf16")
    b = ref.round_to(rng.standard_normal((K, N), dtype=np.float32) / np.float32(np.sqrt(K)), "bf16")
    c, path = tmtest.run_matmul(a, b, "bf16")
    assert path == cuda.PATH_TCGEN05
    rows = np.r_[0:32, 8000:8032, M - 32:M]
    assert ref.relative_error(c[rows], ref.matmul(a[rows], b)) <= 2e-2


def test_launch_validation_on_the_device(core):
    """Errors the reference raises at dispatch (Runtime.swift:201-211) plus the
    host-side extent check that stands in for a memory sanitizer."""
    from triton_metal import kernels
    mm = kernels.Matmul("f32", (64, 64, 16))
    a = tmtest.empty((64, 64), "f32")
    try:
        grid, kinds, values = mm.arguments(a.tm_handle, a.tm_handle, a.tm_handle, 64, 64, 64)
        with pytest.raises(RuntimeError, match="grid must be positive"):
            core.launch(mm.handle, (0, 1, 1), 128, kinds, values)
        with pytest.raises(RuntimeError, match="threadsPerThreadgroup must be positive"):
            core.launch(mm.handle, grid, 0, kinds, values)
        with pytest.raises(RuntimeError, match="exceeds the pipeline maximum"):
            core.launch(mm.handle, grid, 2048, kinds, values)
        big = list(values)
        big[3] = 128                                     # M = 128 rows of a 64-row buffer
        with pytest.raises(RuntimeError, match="beyond its"):
            core.launch(mm.handle, (2, 1, 1), 128, kinds, big)
        kinds_bad = list(kinds)
        kinds_bad[0] = 1
        with pytest.raises(RuntimeError, match="is a pointer"):
            core.launch(mm.handle, grid, 128, kinds_bad, values)
        # extents and strides of 2^32 carried as i64: their product does not fit 64 bits and
        # must be refused, not wrapped into something that looks in bounds
        wide_kinds, wide = list(kinds), list(values)
        for position in (3, 6):                          # M and stride_am
            wide_kinds[position] = core.ARG_I64
            wide[position] = 1 << 32
        with pytest.raises(RuntimeError, match="above 2\\^31|beyond its"):
            core.launch(mm.handle, (1 << 26, 1, 1), 128, wide_kinds, wide)
        wide[3] = 64
        wide[6] = 1 << 62                                # (M-1) * stride_am = 63 * 2^62
        with pytest.raises(RuntimeError, match="beyond its"):
            core.launch(mm.handle, grid, 128, wide_kinds, wide)
    finally:
        mm.release()
        a.free()


@pytest.mark.parametrize("shape", [(256, 256, 256), (384, 200, 1000), (1024, 512, 4096), (130, 72, 520)])
def test_fp32_tensor_core_path_is_3xtf32_accurate(shape):
    """fp32 operands on the tensor cores (split into tf32 hi/lo, three MMAs per K
    step, K accumulated in chunks): within 1e-5 of a float64 product for every K."""
    M, N, K = shape
    a, b = inputs.gemm_uniform(M, N, K, seed=K)
    c, path = tmtest.run_matmul(a, b, "f32", path=cuda.PATH_TCGEN05)
    assert path == cuda.PATH_TCGEN05
    want = a.astype(np.float64) @ b.astype(np.float64)
    assert ref.relative_error(c, want) <= 1e-5
    assert ref.relative_error(c, ref.matmul(a, b)) <= 1e-5


def test_fp32_tensor_core_path_takes_any_stride():
    """The operand split rewrites A and B densely, so transposed and padded inputs and a
    strided C all go through the tensor-core path."""
    M, N, K = 256, 192, 320
    a, b = inputs.gemm_normal(M, N, K, seed=4)
    a_t = np.ascontiguousarray(a.T)                    # stride_am = 1, stride_ak = M
    b_pad = np.zeros((K, N + 5), dtype=np.float32)
    b_pad[:, :N] = b
    strides = (1, M, N + 5, 1, N + 3, 1)
    ab, bb = tmtest.upload(a_t, "f32"), tmtest.upload(b_pad, "f32")
    cb = tmtest.empty((M, N + 3), "f32")
    tmtest.put(cb, np.full((M, N + 3), -9.0, dtype=np.float32))
    from triton_metal import kernels
    mm = kernels.Matmul("f32", (128, 128, 32))
    try:
        mm.set_path(cuda.PATH_TCGEN05)
        mm(ab.tm_handle, bb.tm_handle, cb.tm_handle, M, N, K, strides)
        c = tmtest.fetch(cb)
        assert mm.last_path() == cuda.PATH_TCGEN05
        assert ref.relative_error(c[:, :N], ref.matmul(a, b)) <= 1e-5
        assert np.all(c[:, N:] == -9.0)
    finally:
        mm.release()
        for buf in (ab, bb, cb):
            buf.free()


def test_fp32_large_k_against_float64_rows():
    M, N, K = 512, 2048, 8192
    a, b = inputs.gemm_normal(M, N, K, seed=12)
    c, path = tmtest.run_matmul(a, b, "f32")
    assert path == cuda.PATH_TCGEN05
    rows = np.r_[0:16, 250:266, M - 16:M]
    want = a[rows].astype(np.float64) @ b.astype(np.float64)
    assert ref.relative_error(c[rows], want) <= 1e-5


def test_device_only_buffers(core):
    """tmx_alloc_device_buffer: plain device memory that kernels and copies use like any
    other buffer, but that has no host pointer."""
    n = 256
    a, b = inputs.gemm_normal(n, n, n, seed=6)
    a, b = ref.round_to(a, "bf16"), ref.round_to(b, "bf16")
    ab, bb = tmtest.upload(a, "bf16"), tmtest.upload(b, "bf16")
    c = cuda.alloc_device_buffer(n * n * 2)
    from triton_metal import kernels
    mm = kernels.Matmul("bf16")
    try:
        assert cuda.device_pointer(c) % 256 == 0
        assert core.buffer_length(c) == n * n * 2
        with pytest.raises(RuntimeError, match="device-only"):
            core.buffer_contents(c)
        mm(ab.tm_handle, bb.tm_handle, c, n, n, n)
        out = np.empty((n, n), dtype=ref.storage_dtype("bf16"))
        core.buffer_read(c, 0, out.ctypes.data, out.nbytes)
        assert ref.relative_error(out.astype(np.float32), ref.matmul(a, b)) <= 2e-2
    finally:
        mm.release()
        core.free_buffer(c)
        ab.free()
        bb.free()


def test_pipelined_pieces_with_side_stream_read_back(core):
    """Asynchronous writes and launches on the library's stream, read-backs on its side stream:
    four row pieces in flight give the same C as one blocking launch, and tmx_synchronize /
    tmx_timer_end wait for the read-backs."""
    from triton_metal import kernels
    m, n, k, pieces = 1024, 512, 256, 4
    a, b = inputs.gemm_normal(m, n, k, seed=9)
    a, b = ref.round_to(a, "bf16"), ref.round_to(b, "bf16")
    dt = ref.storage_dtype("bf16")
    a_host, b_host = np.ascontiguousarray(a.astype(dt)), np.ascontiguousarray(b.astype(dt))
    rows = m // pieces
    mm = kernels.Matmul("bf16")
    bb = core.alloc_buffer(b_host.nbytes)
    a_bufs = [core.alloc_buffer(rows * k * 2) for _ in range(pieces)]
    c_bufs = [cuda.alloc_device_buffer(rows * n * 2) for _ in range(pieces)]
    outs = [np.zeros((rows, n), dtype=dt) for _ in range(pieces)]
    parts = [np.ascontiguousarray(a_host[i * rows:(i + 1) * rows]) for i in range(pieces)]
    try:
        for rounds in range(2):                       # the second round reuses every buffer
            cuda.timer_begin()
            cuda.write_async(bb, 0, b_host.ctypes.data, b_host.nbytes)
            for i in range(pieces):
                cuda.write_async(a_bufs[i], 0, parts[i].ctypes.data, parts[i].nbytes)
                mm.launch_async(*mm.arguments(a_bufs[i], bb, c_bufs[i], rows, n, k))
                cuda.read_async(c_bufs[i], 0, outs[i].ctypes.data, outs[i].nbytes)
            assert cuda.timer_end() > 0               # waits for the side stream as well
            got = np.concatenate(outs).astype(np.float32)
            assert ref.relative_error(got, ref.matmul(a, b)) <= 2e-2
            for o in outs:
                o[:] = 0
        whole, _ = tmtest.run_matmul(a, b, "bf16", (128, 256, 64))
        cuda.write_async(bb, 0, b_host.ctypes.data, b_host.nbytes)
        for i in range(pieces):
            cuda.write_async(a_bufs[i], 0, parts[i].ctypes.data, parts[i].nbytes)
            mm.launch_async(*mm.arguments(a_bufs[i], bb, c_bufs[i], rows, n, k))
            cuda.read_async(c_bufs[i], 0, outs[i].ctypes.data, outs[i].nbytes)
        cuda.synchronize()
        assert np.array_equal(np.concatenate(outs).astype(np.float32), whole)
    finally:
        mm.release()
        for h in [bb] + a_bufs + c_bufs:
            core.free_buffer(h)


def test_async_write_keeps_its_place_behind_a_launch_that_reads_the_buffer(core):
    """tmx_buffer_write_async runs on a stream of its own, ahead of kernels enqueued before it -
    except the last launch that took the buffer: a new A uploaded right behind a matmul must not
    reach the device before that matmul has read the old one.  Four rounds, each overwriting A
    while the product of the previous A may still be running; every C is checked bit for bit
    against a run with blocking copies."""
    from triton_metal import kernels
    m, n, k = 2048, 2048, 4096
    dt = ref.storage_dtype("bf16")
    mm = kernels.Matmul("bf16")
    a_buf, b_buf = core.alloc_buffer(m * k * 2), core.alloc_buffer(k * n * 2)
    c_bufs = [cuda.alloc_device_buffer(m * n * 2) for _ in range(4)]
    try:
        _, b = inputs.gemm_normal(m, n, k, seed=21)
        b_host = np.ascontiguousarray(ref.round_to(b, "bf16").astype(dt))
        a_hosts = []
        for i in range(4):
            a, _ = inputs.gemm_normal(m, n, k, seed=30 + i)
            a_hosts.append(np.ascontiguousarray(ref.round_to(a, "bf16").astype(dt)))
        cuda.write_async(b_buf, 0, b_host.ctypes.data, b_host.nbytes)
        for i in range(4):
            cuda.write_async(a_buf, 0, a_hosts[i].ctypes.data, a_hosts[i].nbytes)
            mm.launch_async(*mm.arguments(a_buf, b_buf, c_bufs[i], m, n, k))
        cuda.synchronize()
        got = []
        for c in c_bufs:
            out = np.zeros((m, n), dtype=dt)
            core.buffer_read(c, 0, out.ctypes.data, out.nbytes)
            got.append(out.view(np.uint16).copy())
        for i in range(4):
            core.buffer_write(a_buf, 0, a_hosts[i].ctypes.data, a_hosts[i].nbytes)
            mm.launch(*mm.arguments(a_buf, b_buf, c_bufs[0], m, n, k))
            want = np.zeros((m, n), dtype=dt)
            core.buffer_read(c_bufs[0], 0, want.ctypes.data, want.nbytes)
            assert np.array_equal(got[i], want.view(np.uint16)), f"round {i}"
    finally:
        mm.release()
        for h in [a_buf, b_buf] + c_bufs:
            core.free_buffer(h)


def test_launch_waits_for_a_read_back_of_its_output(core):
    """A read-back runs on a side stream; a later launch that writes the same buffer waits for it.
    C of the first product is read back (pinned host memory, so the copy really is asynchronous)
    while a second product into the same C is already enqueued: the host must still receive the
    first product, then the second."""
    import torch
    from triton_metal import kernels
    m, n, k = 4096, 4096, 512
    dt = ref.storage_dtype("bf16")
    mm = kernels.Matmul("bf16")
    a_bufs = [core.alloc_buffer(m * k * 2) for _ in range(2)]
    b_buf, c_buf = core.alloc_buffer(k * n * 2), cuda.alloc_device_buffer(m * n * 2)
    outs = [torch.empty(m * n * 2, dtype=torch.uint8, pin_memory=True) for _ in range(2)]
    try:
        _, b = inputs.gemm_normal(m, n, k, seed=41)
        b_host = np.ascontiguousarray(ref.round_to(b, "bf16").astype(dt))
        core.buffer_write(b_buf, 0, b_host.ctypes.data, b_host.nbytes)
        for i in range(2):
            a, _ = inputs.gemm_normal(m, n, k, seed=50 + i)
            a_host = np.ascontiguousarray(ref.round_to(a, "bf16").astype(dt))
            core.buffer_write(a_bufs[i], 0, a_host.ctypes.data, a_host.nbytes)
        for i in range(2):
            mm.launch_async(*mm.arguments(a_bufs[i], b_buf, c_buf, m, n, k))
            cuda.read_async(c_buf, 0, outs[i].data_ptr(), outs[i].numel())
        cuda.synchronize()
        for i in range(2):
            mm.launch(*mm.arguments(a_bufs[i], b_buf, c_buf, m, n, k))
            want = np.zeros(m * n, dtype=np.uint16)
            core.buffer_read(c_buf, 0, want.ctypes.data, want.nbytes)
            assert np.array_equal(outs[i].numpy().view(np.uint16), want), f"product {i}"
    finally:
        mm.release()
        for h in a_bufs + [b_buf, c_buf]:
            core.free_buffer(h)


def test_async_write_behind_a_launch_older_than_the_event_ring(core):
    """The upload stream waits for the event of the last launch that took the buffer; only the last
    64 launches keep theirs.  A buffer last used 100 launches ago falls back to waiting for
    everything enqueued so far - its new contents must still arrive after that old launch and
    before the next one that reads it."""
    from triton_metal import kernels
    n = 1 << 22
    copy = kernels.Elementwise("copy")
    src, mid, out, other_in, other_out = (core.alloc_buffer(4 * n) for _ in range(5))
    first = np.arange(n, dtype=np.float32)
    second = first[::-1].copy()
    try:
        core.buffer_write(src, 0, first.ctypes.data, first.nbytes)
        core.buffer_write(other_in, 0, first.ctypes.data, first.nbytes)
        copy.launch_async(*copy.arguments(src, mid, n=n))             # reads src
        for _ in range(100):                                          # pushes that launch out of the ring
            copy.launch_async(*copy.arguments(other_in, other_out, n=n))
        cuda.write_async(src, 0, second.ctypes.data, second.nbytes)   # must not land before the first copy
        copy.launch_async(*copy.arguments(src, out, n=n))             # must see the new contents
        cuda.synchronize()
        got_mid, got_out = np.empty(n, dtype=np.float32), np.empty(n, dtype=np.float32)
        core.buffer_read(mid, 0, got_mid.ctypes.data, got_mid.nbytes)
        core.buffer_read(out, 0, got_out.ctypes.data, got_out.nbytes)
        assert np.array_equal(got_mid, first)
        assert np.array_equal(got_out, second)
    finally:
        copy.release()
        for h in (src, mid, out, other_in, other_out):
            core.free_buffer(h)
