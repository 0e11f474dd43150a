"""The path a launch takes when a wait inside a kernel runs out, in the two forms that fault
nothing: a status record written from the host, and a kernel whose waits are meant to run out.

Every wait inside the tensor-core kernels is bounded by a cycle budget; when it runs out the
kernel writes a record (site, block, detail) into host-visible memory and returns, and the
next synchronising call returns -1 with "a bounded wait gave up inside the kernel", clears
the record and leaves the context usable.  The real kernels cannot be made to time out without
breaking one, so the record comes from `tmx_debug_inject_status` (host) and from
`tmx_selftest_bounded_wait` (a small kernel that waits, with the same wait routines and a
budget of about a millisecond, on a barrier nothing arrives on, and then returns normally)."""

import numpy as np
import pytest

import tmtest
from oracle import reference_math as ref
from triton_metal import _core, cuda, kernels
from triton_metal.buffer import MetalBuffer

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _gpu():
    tmtest.require_gpu()


def small_add():
    n = 4096
    a = np.arange(n, dtype=np.float32)
    bufs = [MetalBuffer.from_numpy(a), MetalBuffer.from_numpy(a), MetalBuffer((n,), "float32")]
    add = kernels.Elementwise("add", 1024)
    return add, bufs, a


def test_injected_status_fails_the_next_launch_and_is_cleared():
    add, bufs, a = small_add()
    try:
        cuda.inject_status(1, 36, 17, 1)
        with pytest.raises(RuntimeError, match=r"a bounded wait gave up inside the kernel \(code 1, site 36, "
                                               r"block 17, detail 1\); the results of this launch are not valid"):
            add(*(b.tm_handle for b in bufs), n=a.size)
        assert _core.last_error() == "no error"              # reading the error cleared the slot
        add(*(b.tm_handle for b in bufs), n=a.size)           # the record was cleared: this one passes
        assert np.array_equal(bufs[2].numpy(), a + a)
        cuda.inject_status(1, 2, 0, 0)
        with pytest.raises(RuntimeError, match="a bounded wait gave up"):
            cuda.synchronize()
        cuda.synchronize()
    finally:
        add.release()
        for b in bufs:
            b.free()


def test_a_wait_that_runs_out_is_reported_and_the_context_stays_usable():
    add, bufs, a = small_add()
    try:
        # 2,000,000 cycles: about a millisecond
        thread_wait, warp_wait = cuda.selftest_bounded_wait(2_000_000)
        assert (thread_wait, warp_wait) == (1, 1)             # both forms of the wait gave up
        with pytest.raises(RuntimeError, match=r"a bounded wait gave up inside the kernel \(code 1, site 9[01], "
                                               r"block 0"):
            cuda.synchronize()
        cuda.synchronize()                                    # cleared
        # the same context goes on computing, on the tensor cores too
        add(*(b.tm_handle for b in bufs), n=a.size)
        assert np.array_equal(bufs[2].numpy(), a + a)
        x = ref.round_to(np.random.default_rng(0).standard_normal((256, 256), dtype=np.float32) / 16, "bf16")
        c, path = tmtest.run_matmul(x, x, "bf16")
        assert path == cuda.PATH_TCGEN05
        assert ref.relative_error(c, ref.matmul(x, x)) <= 2e-2
    finally:
        add.release()
        for b in bufs:
            b.free()


def test_selftest_argument_validation():
    with pytest.raises(RuntimeError, match="budget of 1...2e9"):
        cuda.selftest_bounded_wait(0)
    with pytest.raises(RuntimeError, match="budget of 1...2e9"):
        cuda.selftest_bounded_wait(3_000_000_000)
