"""The plugin's launch marshalling replayed over libtmcuda.

python/plugin/backend/driver.py:58-92 (`MetalLauncher.__call__`) builds `kinds[]` / `values[]`
from the `metal_args` of `tm_kernel_info` (python/plugin/backend/compiler.py:131-146):
a position map over the non-constexpr parameters of the Python call, `tm_handle` on pointer
arguments or TypeError, f32 as its bit pattern (kind 2), i1...i32 as kind 1, i64 as kind 3,
anything else TypeError.  `triton_metal.launcher` restates that; the host-side tests check the
arrays it produces (and, when a reference checkout is at hand, that the reference's own
launcher produces the same arrays from the same metadata); the GPU tests launch
`matmul_kernel` in its nine-argument folded-stride form and `attn_fwd` in both argument
orders through it and compare with the oracle.
"""

import os
import sys
from pathlib import Path

import numpy as np
import pytest

import tmtest
from oracle import inputs, reference_math as ref
from triton_metal import _core, kernels, launcher
from triton_metal.buffer import MetalBuffer

REFERENCE = Path(os.environ.get("TRITON_METAL_REFERENCE") or "/nonexistent-reference-checkout")

#: Triton's `src.signature` of python/examples/matmul.py's kernel for a row-major call: the
#: three unit strides and the three block sizes are specialised away.
MATMUL_SIGNATURE = {
    "a_ptr": "*fp32", "b_ptr": "*fp32", "c_ptr": "*fp32", "M": "i32", "N": "i32", "K": "i32",
    "stride_am": "i32", "stride_ak": "constexpr", "stride_bk": "i32", "stride_bn": "constexpr",
    "stride_cm": "i32", "stride_cn": "constexpr", "BLOCK_SIZE_M": "constexpr",
    "BLOCK_SIZE_N": "constexpr", "BLOCK_SIZE_K": "constexpr",
}


class FakeBuffer:
    def __init__(self, handle):
        self.tm_handle = handle


def matmul_call(a, b, c, M, N, K, block):
    """The positional arguments of `matmul_kernel[grid](...)` in python/examples/matmul.py:55-62."""
    return (a, b, c, M, N, K, K, 1, N, 1, N, 1, *block)


# ---------------------------------------------------------------------------- host side

@pytest.mark.parametrize("positional", [False, True])
def test_folded_matmul_is_marshalled_from_kernel_info(positional):
    ir = kernels.matmul_ir(64, 32, 16, "f32", fold_unit_strides=True, positional_names=positional)
    metadata, image = launcher.make_msl(ir, 4)
    assert metadata["name"] == "matmul_kernel" and metadata["block_shape"] == [64, 32]
    assert [kind for _, kind, _ in metadata["metal_args"]] == ["pointer"] * 3 + ["scalar"] * 6
    assert [dtype for _, _, dtype in metadata["metal_args"]] == ["f32"] * 3 + ["i32"] * 6
    lau = launcher.Launcher(MATMUL_SIGNATURE)
    assert lau.positions == [0, 1, 2, 3, 4, 5, 6, 8, 10]
    call = matmul_call(FakeBuffer(11), FakeBuffer(12), FakeBuffer(13), 300, 200, 100, (64, 32, 16))
    kinds, values = lau.marshal(metadata["metal_args"], call)
    assert kinds == [0, 0, 0, 1, 1, 1, 1, 1, 1]
    # stride_am = K, stride_bk = N, stride_cm = N: the unit strides at call positions 7, 9, 11 are skipped
    assert values == [11, 12, 13, 300, 200, 100, 100, 200, 200]


def test_scalar_kinds_and_type_errors():
    ir = """module {
  tt.func public @attn_fwd(%Q: !tt.ptr<f16>, %K: !tt.ptr<f16>, %V: !tt.ptr<f16>, %O: !tt.ptr<f16>,
      %sm_scale: f32, %stride_head: i64, %stride_seq: i32, %n_ctx: i32) {
    %s = tt.dot %x, %y, %z : tensor<32x64xf16> * tensor<64x32xf16> -> tensor<32x32xf32>
    tt.return
  }
}
"""
    metadata, _ = launcher.make_msl(ir)
    lau = launcher.Launcher({f"p{i}": "x" for i in range(8)})
    bufs = [FakeBuffer(h) for h in (5, 6, 7, 8)]
    kinds, values = lau.marshal(metadata["metal_args"], (*bufs, 0.125, 1 << 33, 64, 96))
    assert kinds == [0, 0, 0, 0, _core.ARG_F32, _core.ARG_I64, _core.ARG_I32, _core.ARG_I32]
    assert values[4] == 0x3E000000 and values[5] == 1 << 33
    # a pointer argument that is not device memory
    with pytest.raises(TypeError, match="argument 1 .*ndarray.* not backed by device memory"):
        lau.marshal(metadata["metal_args"], (bufs[0], np.zeros(4), bufs[2], bufs[3], 0.125, 1, 64, 96))
    # a scalar type the ABI does not carry (the scan refuses f64 by itself, so the launcher is
    # given the metadata directly)
    bad = list(metadata["metal_args"])
    bad[4] = (4, "scalar", "f64")
    with pytest.raises(TypeError, match="argument 4 has scalar type 'f64'"):
        lau.marshal(bad, (*bufs, 0.125, 1, 64, 96))


@pytest.mark.skipif(not REFERENCE.exists(), reason="set TRITON_METAL_REFERENCE to a reference checkout")
def test_the_reference_launcher_builds_the_same_arrays(monkeypatch):
    """The reference's own MetalLauncher (imported unmodified, its `_core` bound to libtmcuda)
    and the restatement here, fed the same metadata and call."""
    pytest.importorskip("triton")
    monkeypatch.syspath_prepend(str(REFERENCE / "python" / "plugin"))
    try:
        from backend import driver as ref_driver
    except Exception as exc:      # a Triton too old for the plugin's imports
        pytest.skip(f"the reference plugin does not import here: {exc}")
    seen = {}
    monkeypatch.setattr(ref_driver._core, "launch",
                        lambda fn, grid, threads, kinds, values: seen.update(
                            fn=fn, grid=grid, threads=threads, kinds=list(kinds), values=list(values)))

    class Src:
        signature = MATMUL_SIGNATURE

    for ir, call in (
        (kernels.matmul_ir(64, 32, 16, "f32", fold_unit_strides=True),
         matmul_call(FakeBuffer(1), FakeBuffer(2), FakeBuffer(3), 256, 128, 64, (64, 32, 16))),
    ):
        metadata, _ = launcher.make_msl(ir, 4)
        theirs = ref_driver.MetalLauncher(Src, metadata)
        packed = (4, metadata["threads_per_threadgroup"], metadata["metal_args"])
        theirs(4, 4, 1, 0, 77, packed, None, None, None, *call)
        ours = launcher.Launcher(MATMUL_SIGNATURE)
        kinds, values = ours.marshal(metadata["metal_args"], call)
        assert theirs.positions == ours.positions
        assert (seen["kinds"], seen["values"]) == (kinds, values)
        assert seen["threads"] == metadata["threads_per_threadgroup"] and seen["fn"] == 77


def test_kernel_wrappers_marshal_through_kernel_info():
    """`kernels.*` builds its arrays from the JSON too: a matmul's arrays equal the launcher's."""
    mm = kernels.Matmul("bf16", (128, 256, 64))
    try:
        _, kinds, values = mm.arguments(3, 4, 5, 512, 256, 128)
        assert kinds == [0, 0, 0] + [1] * 9
        assert values == [3, 4, 5, 512, 256, 128, 128, 1, 256, 1, 256, 1]
        assert [d for _, _, d in mm.metal_args][:3] == ["bf16"] * 3
    finally:
        mm.release()


# ---------------------------------------------------------------------------- on the GPU

@pytest.mark.gpu
@pytest.mark.parametrize("positional", [False, True])
def test_folded_matmul_launches_through_the_replay(positional):
    tmtest.require_gpu()
    M, N, K, block = 256, 256, 256, (64, 64, 32)
    rng = np.random.default_rng(0)
    a = rng.uniform(-1, 1, (M, K)).astype(np.float32)
    b = rng.uniform(-1, 1, (K, N)).astype(np.float32)
    compiled = launcher.CompiledKernel(
        kernels.matmul_ir(*block, "f32", fold_unit_strides=True, positional_names=positional),
        MATMUL_SIGNATURE)
    bufs = [MetalBuffer.from_numpy(a), MetalBuffer.from_numpy(b), MetalBuffer((M, N), "float32")]
    try:
        grid = (kernels.cdiv(M, block[0]), kernels.cdiv(N, block[1]))
        compiled[grid](*matmul_call(*bufs, M, N, K, block))
        assert ref.relative_error(bufs[2].numpy(), ref.matmul(a, b)) <= 1e-5
        with pytest.raises(TypeError, match="not backed by device memory"):
            compiled[grid](*matmul_call(a, bufs[1], bufs[2], M, N, K, block))
    finally:
        compiled.release()
        for buf in bufs:
            buf.free()


@pytest.mark.gpu
@pytest.mark.parametrize("order", ["python", "swift", "swift_no_stats"])
def test_attn_fwd_in_both_argument_orders(order):
    tmtest.require_gpu()
    bh, seq, d = 2, 96, 64
    q, k, v, _ = inputs.attention_normal(bh, seq, d, seed=3)
    scale = ref.default_scale(d)
    compiled = launcher.CompiledKernel(kernels.attn_fwd_ir(16, 32, d, "f32", order=order),
                                       {f"p{i}": "x" for i in range(8 if order == "swift_no_stats" else 10)})
    bufs = {n: MetalBuffer.from_numpy(t) for n, t in (("q", q), ("k", k), ("v", v))}
    bufs["o"] = MetalBuffer((bh, seq, d), "float32")
    bufs["l"] = MetalBuffer((bh, seq), "float32")
    try:
        grid = (kernels.cdiv(seq, 16), bh)
        if order == "python":     # python/examples/attention_training.py:38
            call = (bufs["q"], bufs["k"], bufs["v"], bufs["o"], bufs["l"], scale, seq * d, d, seq, seq)
        elif order == "swift":    # Sources/TritonMetalBench/AttentionKernel.swift:75-78
            call = (bufs["q"], bufs["k"], bufs["v"], bufs["o"], scale, seq * d, d, seq, bufs["l"], seq)
        else:
            call = (bufs["q"], bufs["k"], bufs["v"], bufs["o"], scale, seq * d, d, seq)
        compiled[grid](*call)
        want, _ = ref.attention_forward(q, k, v, scale)
        assert ref.relative_error(bufs["o"].numpy(), want) <= 1e-5
        if order != "swift_no_stats":
            assert np.max(np.abs(bufs["l"].numpy() - ref.logsumexp_log2(q, k, scale))) <= 1e-4
    finally:
        compiled.release()
        for buf in bufs.values():
            buf.free()
