"""Parity at the full sizes of the benchmark configurations, through the C ABI.

The oracle is quadratic in the sequence length, so at these sizes it is evaluated on samples:
blocks of query rows of a few (batch, head) slices for the forward (the first rows, a block
that straddles the middle, the last rows of the last head - where a 32-bit offset or a phase
counter that wrapped would show), whole heads for the backward at S = 4096, row blocks and a
checksum of checksums (column sums) for the 8192^3 GEMM.  Every output is also scanned for
values that are not finite and for heads that were never written.

Tolerances: the 16-bit bound of the benchmark configurations (2e-2 with the reference's
`relative_error`, python/examples/attention_training.py:250-252) and, beside it, the bounds the
reference's own tests hold for 16-bit matmuls - |a-b| / max(1, |b|) below 2^-8 for bf16
(Tests/TritonMetalCoreTests/DotTests.swift:514-554) and 5e-3 for f16 (:466-506) - and 4e-3 for
f16 attention (Tests/TritonMetalCoreTests/AttentionTests.swift:140-150).
"""

import numpy as np
import pytest

import tmtest
from oracle import inputs, reference_math as ref
from triton_metal import _core, cuda, kernels
from triton_metal.synthetic import attention_inputs_bf16, from_bf16_bits, gemm_inputs_bf16

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _gpu():
    tmtest.require_gpu()


def dot_test_error(got, want):
    """max |a - b| / max(1, |b|): the metric of the reference's 16-bit matmul tests."""
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    return float(np.max(np.abs(got - want) / np.maximum(1.0, np.abs(want))))


def every_slice_written(bits, slices):
    """No NaN/inf anywhere and no (batch, head) slice left at zero, from the bf16 words."""
    mag = (bits & np.uint16(0x7FFF)).reshape(slices, -1)
    per_slice = mag.max(axis=1)
    return bool(np.all(per_slice < 0x7F80) and np.all(per_slice > 0))


class DeviceTensors:
    """Named plain-device buffers filled from bf16 words; read back as words."""

    def __init__(self):
        self.handles, self.sizes = {}, {}

    def put(self, name, bits):
        self.alloc(name, bits.nbytes)
        _core.buffer_write(self.handles[name], 0, bits.ctypes.data, bits.nbytes)

    def alloc(self, name, nbytes):
        self.handles[name] = cuda.alloc_device_buffer(nbytes)
        self.sizes[name] = nbytes

    def __getitem__(self, name):
        return self.handles[name]

    def words(self, name, shape, dtype=np.uint16):
        out = np.empty(shape, dtype=dtype)
        assert out.nbytes == self.sizes[name]
        _core.buffer_read(self.handles[name], 0, out.ctypes.data, out.nbytes)
        return out

    def close(self):
        for h in self.handles.values():
            _core.free_buffer(h)
        self.handles = {}


# --------------------------------------------------------------------------- forward

def check_forward_samples(host, o_bits, lse, causal, heads, row_blocks, tol=2e-2):
    seq, d = host[0].shape[1:]
    scale = ref.default_scale(d)
    for h in heads:
        q, k, v = (from_bf16_bits(t[h]) for t in host)
        for r0, r1 in row_blocks:
            keys = r1 if causal else seq          # later keys are masked for every row of the block
            want, _ = ref.attention_forward(q[r0:r1], k[:keys], v[:keys], scale, causal, row0=r0)
            got = from_bf16_bits(o_bits[h, r0:r1])
            assert ref.relative_error(got, want) <= tol, (h, r0)
            want_lse = ref.logsumexp_log2(q[r0:r1], k[:keys], scale, causal, row0=r0)
            assert np.max(np.abs(lse[h, r0:r1] - want_lse)) <= 2e-2, (h, r0)


@pytest.fixture(scope="module")
def long_sequence_inputs():
    """Batch 4, heads 32, seq 16384, head_dim 128: 512 MiB per tensor, made once for both masks."""
    bh, seq, d = 128, 16384, 128
    host = attention_inputs_bf16(bh, seq, d, seed=16384, count=3)
    dev = DeviceTensors()
    for name, bits in zip(("q", "k", "v"), host):
        dev.put(name, bits)
    dev.alloc("o", bh * seq * d * 2)
    dev.alloc("lse", bh * seq * 4)
    yield host, dev
    dev.close()


@pytest.mark.parametrize("causal", [True, False])
def test_forward_b4_h32_s16384_d128(long_sequence_inputs, causal):
    host, dev = long_sequence_inputs
    bh, seq, d = host[0].shape
    fwd = kernels.AttnFwd("bf16", d, (128, 128), causal)
    try:
        fwd.set_path(cuda.PATH_TCGEN05)
        cuda.fill(dev["o"], 0, 0, bh * seq * d * 2)
        fwd(dev["q"], dev["k"], dev["v"], dev["o"], dev["lse"], ref.default_scale(d), bh, seq)
        o_bits = dev.words("o", (bh, seq, d))
        lse = dev.words("lse", (bh, seq), np.float32)
    finally:
        fwd.release()
    assert every_slice_written(o_bits, bh)
    assert np.all(np.isfinite(lse))
    blocks = [(0, 128), (seq // 2 - 128, seq // 2 + 128), (seq - 256, seq)]
    check_forward_samples(host, o_bits, lse, causal, [0, 61, bh - 1], blocks)


@pytest.mark.parametrize("seq", [1024, 4096])
@pytest.mark.parametrize("causal", [True, False])
def test_forward_b4_h32_d128(seq, causal):
    bh, d = 128, 128
    host = attention_inputs_bf16(bh, seq, d, seed=seq, count=3)
    dev = DeviceTensors()
    fwd = kernels.AttnFwd("bf16", d, (128, 128), causal)
    try:
        for name, bits in zip(("q", "k", "v"), host):
            dev.put(name, bits)
        dev.alloc("o", bh * seq * d * 2)
        dev.alloc("lse", bh * seq * 4)
        fwd.set_path(cuda.PATH_TCGEN05)
        fwd(dev["q"], dev["k"], dev["v"], dev["o"], dev["lse"], ref.default_scale(d), bh, seq)
        o_bits = dev.words("o", (bh, seq, d))
        lse = dev.words("lse", (bh, seq), np.float32)
    finally:
        fwd.release()
        dev.close()
    assert every_slice_written(o_bits, bh)
    check_forward_samples(host, o_bits, lse, causal, [0, 50, bh - 1], [(0, seq)])


# --------------------------------------------------------------------------- backward

@pytest.mark.parametrize("d", [64, 128])
def test_backward_b8_h16_s4096_causal(d):
    bh, seq, causal = 128, 4096, True
    host = attention_inputs_bf16(bh, seq, d, seed=4096 + d, count=4)
    scale = ref.default_scale(d)
    dev = DeviceTensors()
    kerns = [kernels.AttnFwd("bf16", d, (128, 128), causal), kernels.AttnBwdPreprocess("bf16", d, 128),
             kernels.AttnBwdDq("bf16", d, (128, 128), causal), kernels.AttnBwdDkdv("bf16", d, (128, 128), causal)]
    fwd, pre, dq, dkdv = kerns
    try:
        for name, bits in zip(("q", "k", "v", "do"), host):
            dev.put(name, bits)
        for name in ("o", "dq", "dk", "dv"):
            dev.alloc(name, bh * seq * d * 2)
        for name in ("lse", "delta"):
            dev.alloc(name, bh * seq * 4)
        for kern in (fwd, dq, dkdv):
            kern.set_path(cuda.PATH_TCGEN05)
        fwd(dev["q"], dev["k"], dev["v"], dev["o"], dev["lse"], scale, bh, seq)
        pre(dev["o"], dev["do"], dev["delta"], bh, seq)
        dq(dev["q"], dev["k"], dev["v"], dev["do"], dev["dq"], dev["lse"], dev["delta"], scale, bh, seq)
        dkdv(dev["q"], dev["k"], dev["v"], dev["do"], dev["dk"], dev["dv"], dev["lse"], dev["delta"],
             scale, bh, seq)
        assert [k.last_path() for k in (fwd, dq, dkdv)] == [cuda.PATH_TCGEN05] * 3
        got = {n: dev.words(n, (bh, seq, d)) for n in ("o", "dq", "dk", "dv")}
    finally:
        for kern in kerns:
            kern.release()
        dev.close()
    for name, bits in got.items():
        assert every_slice_written(bits, bh), name
    for h in (0, 64, bh - 1):
        q, k, v, do = (from_bf16_bits(t[h:h + 1]) for t in host)
        want_o, _, want_dq, want_dk, want_dv = tmtest.oracle_attention(q, k, v, do, causal)
        for name, want in (("o", want_o), ("dq", want_dq), ("dk", want_dk), ("dv", want_dv)):
            assert ref.relative_error(from_bf16_bits(got[name][h:h + 1]), want) <= 2e-2, (name, h)


# --------------------------------------------------------------------------- GEMM

def test_gemm_bf16_8192_cubed():
    n = 8192
    a_bits, b_bits = gemm_inputs_bf16(n, n, n, seed=0)
    dev = DeviceTensors()
    mm = kernels.Matmul("bf16", (128, 256, 64))
    try:
        dev.put("a", a_bits)
        dev.put("b", b_bits)
        dev.alloc("c", n * n * 2)
        mm(dev["a"], dev["b"], dev["c"], n, n, n)
        assert mm.last_path() == cuda.PATH_TCGEN05
        c = from_bf16_bits(dev.words("c", (n, n)))
    finally:
        mm.release()
        dev.close()
    a, b = from_bf16_bits(a_bits), from_bf16_bits(b_bits)
    rows = np.r_[0:64, 4000:4064, n - 64:n]
    want = ref.matmul(a[rows], b)
    # 2e-2 is the configuration's bound; one bf16 rounding of the result (2^-9 of the largest
    # element) is all the error there should be, so the tighter 2^-8 must hold as well
    assert ref.relative_error(c[rows], want) <= 2.0 ** -8
    # checksum of checksums: the column sums of C against (column sums of A) @ B in float64.
    # Each element of C carries one bf16 rounding (relative 2^-9); over 8192 rows the
    # roundings average out, so the sums agree far more closely than the elements do.
    sums = c.astype(np.float64).sum(axis=0)
    want_sums = a.astype(np.float64).sum(axis=0) @ b.astype(np.float64)
    assert np.max(np.abs(sums - want_sums)) <= 2.0 ** -8 * np.sqrt(n) * np.max(np.abs(want))
    assert np.all(np.isfinite(c))


# --------------------------------------------------------------------------- reference-held 16-bit bounds

@pytest.mark.parametrize("element,bound", [("bf16", 2.0 ** -8), ("f16", 5e-3)])
@pytest.mark.parametrize("shape", [(129, 257, 65), (512, 512, 512), (1024, 768, 2048)])
def test_16bit_matmul_meets_the_bounds_of_the_reference_tests(element, bound, shape):
    M, N, K = shape
    # uniform[-1, 1) operands: results of magnitude sqrt(K/3), so the metric is a relative one
    # and a result that was truncated instead of rounded would not pass
    a, b = (ref.round_to(t, element) for t in inputs.gemm_uniform(M, N, K, seed=M + K))
    want = ref.matmul(a, b)
    for path in (cuda.PATH_SIMT, cuda.PATH_AUTO):
        c, _ = tmtest.run_matmul(a, b, element, path=path)
        assert dot_test_error(c, want) <= bound, (element, shape, path)


@pytest.mark.parametrize("bh,seq,d,path", [(2, 96, 64, cuda.PATH_SIMT), (1, 127, 64, cuda.PATH_SIMT),
                                          (2, 512, 64, cuda.PATH_TCGEN05), (2, 640, 128, cuda.PATH_TCGEN05)])
def test_f16_attention_forward_meets_the_bound_of_the_reference_tests(bh, seq, d, path):
    q, k, v, do = (ref.round_to(t, "f16") for t in inputs.attention_normal(bh, seq, d, seed=seq))
    want, _ = ref.attention_forward(q, k, v, ref.default_scale(d))
    block = (128, 128) if path == cuda.PATH_TCGEN05 else (32, 32)
    with tmtest.AttentionRun(q, k, v, do, "f16", False, block, path) as run:
        o, _ = run.forward()
    assert dot_test_error(o, want) <= 4e-3
