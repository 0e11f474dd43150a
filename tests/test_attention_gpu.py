"""attn_fwd / attn_bwd_* parity through the C ABI, against the numpy oracle.

Shapes follow Tests/TritonMetalCoreTests/AttentionTests.swift:119-135 (s127/512/
96/33/64, d64/80), the overflow case :161-177, AttentionBackwardTests.swift and
python/examples/attention_training.py:255-330 (h2 s96 d64, loss must decrease);
tolerances: fp32 1e-5 with the reference's relative_error, 16-bit 2e-2."""

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


def check_all(q, k, v, do, element, causal, block=(128, 128), path=0, tol=None):
    tol = tol or TOL[element]
    q, k, v, do = (ref.round_to(t, element) for t in (q, k, v, do))
    want_o, want_lse, want_dq, want_dk, want_dv = tmtest.oracle_attention(q, k, v, do, causal)
    with tmtest.AttentionRun(q, k, v, do, element, causal, block, path) as run:
        o, lse = run.forward()
        dq, dk, dv = run.backward()
        paths = run.paths()
    assert ref.relative_error(o, want_o) <= tol, "O"
    assert np.max(np.abs(lse - want_lse)) <= (1e-4 if element == "f32" else 2e-2), "LSE"
    for name, got, want in (("dQ", dq, want_dq), ("dK", dk, want_dk), ("dV", dv, want_dv)):
        assert ref.relative_error(got, want) <= tol, name
    return paths


@pytest.mark.parametrize("bh,seq,d", [(2, 96, 64), (1, 127, 64), (1, 512, 64), (3, 33, 80),
                                      (2, 64, 64), (1, 48, 64), (2, 200, 128), (1, 70, 32)])
@pytest.mark.parametrize("causal", [False, True])
def test_fp32_shapes(bh, seq, d, causal):
    q, k, v, do = inputs.attention_normal(bh, seq, d, seed=seq + d)
    check_all(q, k, v, do, "f32", causal, block=(16, 32))


@pytest.mark.parametrize("element", ["f16", "bf16"])
@pytest.mark.parametrize("bh,seq,d", [(2, 96, 64), (1, 127, 64), (2, 33, 80), (2, 256, 128)])
@pytest.mark.parametrize("causal", [False, True])
def test_16bit_shapes(element, bh, seq, d, causal):
    q, k, v, do = inputs.attention_normal(bh, seq, d, seed=seq)
    check_all(q, k, v, do, element, causal, block=(32, 32))


@pytest.mark.parametrize("bh,seq,d,causal,path", [
    (2, 1024, 64, False, cuda.PATH_AUTO), (2, 1024, 64, True, cuda.PATH_AUTO), (1, 2048, 128, True, cuda.PATH_AUTO),
    (2, 1000, 64, True, cuda.PATH_TCGEN05), (3, 300, 80, False, cuda.PATH_TCGEN05),
])
def test_fp32_long_sequences_run_on_the_tensor_cores(bh, seq, d, causal, path):
    """fp32 attention from 1024 rows on (from 256 when the tensor-core path is asked for): every
    contraction of the three kernels as a 3xTF32 GEMM over a materialised score matrix, the
    softmax and dS products as row-wise fp32 kernels.  Same bound as the exact-FMA kernels -
    1e-5 with the reference's relative_error - and agreement with them."""
    q, k, v, do = inputs.attention_normal(bh, seq, d, seed=seq + d)
    paths = check_all(q, k, v, do, "f32", causal, block=(16, 32), path=path)
    assert [paths[n] for n in ("fwd", "dq", "dkdv")] == [cuda.PATH_TCGEN05] * 3
    with tmtest.AttentionRun(q, k, v, do, "f32", causal, (16, 32), cuda.PATH_SIMT) as run:
        o_simt, lse_simt = run.forward()
        grads_simt = run.backward()
    with tmtest.AttentionRun(q, k, v, do, "f32", causal, (16, 32), path) as run:
        o_tc, lse_tc = run.forward()
        grads_tc = run.backward()
    assert ref.relative_error(o_tc, o_simt) <= 1e-5
    assert np.max(np.abs(lse_tc - lse_simt)) <= 1e-4
    for a, b in zip(grads_tc, grads_simt):
        assert ref.relative_error(a, b) <= 1e-5


def test_fp32_tensor_core_attention_leaves_rows_outside_the_grid_alone():
    bh, seq, d = 1, 1024, 64
    q, k, v, do = inputs.attention_normal(bh, seq, d, seed=77)
    want = tmtest.oracle_attention(q, k, v, do, False)
    with tmtest.AttentionRun(q, k, v, do, "f32", False, (128, 128), cuda.PATH_TCGEN05) as run:
        run.forward()                                   # L for every row
        run.kernels["pre"](run.h("o"), run.h("do"), run.h("delta"), run.bh, run.seq)
        for name in ("o", "dq", "dk", "dv"):
            tmtest.put(run.bufs[name], np.full((bh, seq, d), -7.0, dtype=np.float32))
        rows = 3 * 128
        for kern, args in (("fwd", (run.h("q"), run.h("k"), run.h("v"), run.h("o"), run.h("lse"), run.scale, bh, seq)),
                           ("dq", (run.h("q"), run.h("k"), run.h("v"), run.h("do"), run.h("dq"), run.h("lse"),
                                   run.h("delta"), run.scale, bh, seq)),
                           ("dkdv", (run.h("q"), run.h("k"), run.h("v"), run.h("do"), run.h("dk"), run.h("dv"),
                                     run.h("lse"), run.h("delta"), run.scale, bh, seq))):
            grid, kinds, values = run.kernels[kern].arguments(*args)
            run.kernels[kern].launch((3, grid[1], grid[2]), kinds, values)
        got = {n: tmtest.fetch(run.bufs[n]) for n in ("o", "dq", "dk", "dv")}
    for name, ref_value in (("o", want[0]), ("dq", want[2]), ("dk", want[3]), ("dv", want[4])):
        assert ref.relative_error(got[name][:, :rows], ref_value[:, :rows]) <= 1e-5, name
        assert np.all(got[name][:, rows:] == -7.0), name


def test_golden_case_of_the_reference_example():
    """h2 s96 d64 seed 0: the outputs of the reference's own numpy functions."""
    from pathlib import Path
    golden = np.load(Path(__file__).resolve().parent / "golden" / "attention_reference.npz")
    rng = np.random.default_rng(0)
    q, k, v, target = [rng.standard_normal((2, 96, 64), dtype=np.float32) * np.float32(0.5)
                       for _ in range(4)]
    with tmtest.AttentionRun(q, k, v, np.zeros_like(q), "f32", False, (16, 32)) as run:
        o, _ = run.forward()
        assert ref.relative_error(o, golden["h2_s96_d64_seed0.o"]) < 2e-5
        d_out = (golden["h2_s96_d64_seed0.o"] - target).astype(np.float32)
        tmtest.put(run.bufs["do"], d_out)
        dq, dk, dv = run.backward()
    for name, got in (("dq", dq), ("dk", dk), ("dv", dv)):
        assert ref.relative_error(got, golden[f"h2_s96_d64_seed0.{name}"]) < 2e-5, name


def test_overflow_stability():
    """Scores spread over +-12 with scale 1 stay finite
    (AttentionTests.swift:161-177)."""
    q, k, v, do = inputs.attention_normal(1, 64, 64, seed=1)
    q = q * np.float32(12.0 / 8.0)
    k = k * np.float32(12.0 / 8.0)
    paths = check_all(q, k, v, do, "f32", False, block=(16, 32), tol=2e-5)
    assert paths["fwd"] == cuda.PATH_SIMT


def test_rows_outside_the_grid_are_left_alone():
    q, k, v, do = inputs.attention_normal(1, 64, 64, seed=8)
    with tmtest.AttentionRun(q, k, v, do, "f32", False, (16, 32)) as run:
        from triton_metal import _core
        fwd = run.kernels["fwd"]
        grid, kinds, values = fwd.arguments(run.h("q"), run.h("k"), run.h("v"), run.h("o"),
                                            run.h("lse"), run.scale, run.bh, run.seq)
        fwd.launch((2, 1, 1), kinds, values)            # only the first 32 query rows
        o = tmtest.fetch(run.bufs["o"])
    want, _ = ref.attention_forward(q, k, v, ref.default_scale(64))
    assert ref.relative_error(o[:, :32], want[:, :32]) <= 1e-5
    assert np.all(o[:, 32:] == 0)


def test_gradient_descent_on_projection_weights():
    """The small fp32 configuration's training loop: d_model 128 = 2 heads x 64,
    seq 96, weights N(0, 0.02), MSE to an N(0,1) target, 8 SGD steps at lr 1e-3;
    attention forward/backward on the GPU, loss must fall every step and track
    the oracle's trajectory."""
    rng = np.random.default_rng(0)
    seq, d_model, heads = 96, 128, 2
    x = rng.standard_normal((seq, d_model), dtype=np.float32)
    target = rng.standard_normal((seq, d_model), dtype=np.float32)
    w_gpu = [rng.standard_normal((d_model, d_model), dtype=np.float32) * np.float32(0.02)
             for _ in range(4)]
    w_ref = [w.copy() for w in w_gpu]
    scale = ref.default_scale(d_model // heads)
    zeros = np.zeros((heads, seq, d_model // heads), dtype=np.float32)

    with tmtest.AttentionRun(zeros, zeros, zeros, zeros, "f32", False, (16, 32)) as run:
        def gpu_fwd(q, k, v):
            for name, t in (("q", q), ("k", k), ("v", v)):
                tmtest.put(run.bufs[name], np.asarray(t, dtype=np.float32))
            o, _ = run.forward()
            return o, None

        def gpu_bwd(q, k, v, aux, do):
            tmtest.put(run.bufs["do"], np.asarray(do, dtype=np.float32))
            return run.backward()

        ref_fwd, ref_bwd = ref.oracle_attention(scale)
        losses, ref_losses = [], []
        for _ in range(8):
            loss, grads = ref.projection_step(x, w_gpu, target, heads, scale, gpu_fwd, gpu_bwd)
            ref_loss, ref_grads = ref.projection_step(x, w_ref, target, heads, scale, ref_fwd, ref_bwd)
            losses.append(loss)
            ref_losses.append(ref_loss)
            w_gpu = [w - np.float32(1e-3) * g for w, g in zip(w_gpu, grads)]
            w_ref = [w - np.float32(1e-3) * g for w, g in zip(w_ref, ref_grads)]
    assert all(b < a for a, b in zip(losses, losses[1:])), losses
    assert np.allclose(losses, ref_losses, rtol=1e-5)


def test_projection_training_step_runs_on_the_library():
    """The same eight SGD steps with every product on the GPU: the Q/K/V/O projections and
    their transposed gradients through matmul_kernel (transposes as strides), the head split
    through the attention kernels' strides, the updates through scale_bias_kernel and
    add_kernel.  Losses and weights must follow the numpy chain rule step for step."""
    from triton_metal.attention_layer import ProjectionAttention
    rng = np.random.default_rng(0)
    seq, d_model, heads = 96, 128, 2
    x = rng.standard_normal((seq, d_model), dtype=np.float32)
    target = rng.standard_normal((seq, d_model), dtype=np.float32)
    w_ref = [rng.standard_normal((d_model, d_model), dtype=np.float32) * np.float32(0.02)
             for _ in range(4)]
    scale = ref.default_scale(d_model // heads)
    ref_fwd, ref_bwd = ref.oracle_attention(scale)
    layer = ProjectionAttention(x, target, w_ref, heads)
    try:
        losses, ref_losses = [], []
        for step in range(8):
            before = cuda.launch_count()
            losses.append(layer.forward())
            grads = layer.backward()
            layer.sgd(1e-3)
            # 4 + 5 matmuls, 4 attention kernels, 2 + 8 element-wise launches: nothing ran elsewhere
            assert cuda.launch_count() - before == 23
            ref_loss, ref_grads = ref.projection_step(x, w_ref, target, heads, scale, ref_fwd, ref_bwd)
            ref_losses.append(ref_loss)
            for name, got, want in zip(("dWq", "dWk", "dWv", "dWo"), grads, ref_grads):
                assert ref.relative_error(got, want) <= 1e-5, (step, name)
            w_ref = [w - np.float32(1e-3) * g for w, g in zip(w_ref, ref_grads)]
            for got, want in zip(layer.weights(), w_ref):
                assert ref.relative_error(got, want) <= 1e-5, step
    finally:
        layer.close()
    assert all(b < a for a, b in zip(losses, losses[1:])), losses
    assert np.allclose(losses, ref_losses, rtol=1e-5)


def test_gpu_gradients_match_finite_differences():
    """python/examples/attention_training.py:286-310 and
    Tests/TritonMetalCoreTests/AttentionBackwardTests.swift:397-482: the kernels' dQ, dK, dV of
    0.5*||O - T||^2 on h2 s96 d64 against central differences of a float64 forward, which
    know no backward formulas.  Four entries per tensor, bound 1e-4."""
    rng = np.random.default_rng(0)
    q, k, v, target = [rng.standard_normal((2, 96, 64), dtype=np.float32) * np.float32(0.5)
                       for _ in range(4)]
    scale = ref.default_scale(64)
    with tmtest.AttentionRun(q, k, v, np.zeros_like(q), "f32", False, (16, 32)) as run:
        o, _ = run.forward()
        tmtest.put(run.bufs["do"], (o - target).astype(np.float32))
        grads = run.backward()

    def loss(qq, kk, vv):
        out, _ = ref.attention_forward(qq, kk, vv, scale, dtype=np.float64)
        return 0.5 * float(np.sum((out - target.astype(np.float64)) ** 2))

    h, worst = 1e-5, 0.0
    for which, grad in enumerate(grads):
        for _ in range(4):
            idx = tuple(rng.integers(0, s) for s in q.shape)
            plus = [t.astype(np.float64) for t in (q, k, v)]
            minus = [t.copy() for t in plus]
            plus[which][idx] += h
            minus[which][idx] -= h
            numeric = (loss(*plus) - loss(*minus)) / (2 * h)
            worst = max(worst, abs(numeric - float(grad[idx])) / max(1.0, abs(numeric)))
    assert worst < 1e-4, worst


def test_direct_descent_of_the_reference_example():
    """attention_training.py:314-329 - 8 steps on q, k, v at rate 0.5; the loss
    after the last step is below the first."""
    rng = np.random.default_rng(0)
    q, k, v, target = [rng.standard_normal((2, 96, 64), dtype=np.float32) * np.float32(0.5)
                       for _ in range(4)]
    with tmtest.AttentionRun(q, k, v, np.zeros_like(q), "f32", False, (16, 32)) as run:
        def step(q, k, v):
            for name, t in (("q", q), ("k", k), ("v", v)):
                tmtest.put(run.bufs[name], np.asarray(t, dtype=np.float32))
            o, _ = run.forward()
            return o
        first = None
        for _ in range(8):
            o = step(q, k, v)
            loss = 0.5 * float(np.sum((o - target) ** 2))
            first = loss if first is None else first
            tmtest.put(run.bufs["do"], (o - target).astype(np.float32))
            dq, dk, dv = run.backward()
            q, k, v = q - 0.5 * dq, k - 0.5 * dk, v - 0.5 * dv
        final = 0.5 * float(np.sum((step(q, k, v) - target) ** 2))
    assert final < first


def test_attention_argument_validation(core):
    from triton_metal import kernels
    fwd = kernels.AttnFwd("f32", 64, (16, 32))
    small = tmtest.empty((1, 16, 64), "f32")
    stat = tmtest.empty((1, 16), "f32")
    try:
        grid, kinds, values = fwd.arguments(small.tm_handle, small.tm_handle, small.tm_handle,
                                            small.tm_handle, stat.tm_handle, 0.125, 1, 32)
        with pytest.raises(RuntimeError, match="beyond its"):
            core.launch(fwd.handle, grid, 128, kinds, values)
        pre = kernels.AttnBwdPreprocess("f32", 64)
        with pytest.raises(RuntimeError, match="does not apply"):
            cuda.set_option(pre.handle, "causal", 1)
        pre.release()
    finally:
        fwd.release()
        small.free()
        stat.free()


# ---- the tcgen05 kernels: persistent CTAs, ragged sequences, several work units per CTA ----

@pytest.mark.parametrize("bh,seq,d,causal", [
    (3, 384, 64, True), (2, 1000, 128, True), (2, 1000, 128, False), (5, 2304, 64, False),
    (1, 128, 128, True), (2, 130, 128, False),
])
def test_tensor_core_paths_on_ragged_and_long_sequences(bh, seq, d, causal):
    q, k, v, do = inputs.attention_normal(bh, seq, d, seed=seq + d + causal)
    paths = check_all(q, k, v, do, "bf16", causal, path=cuda.PATH_TCGEN05)
    assert [paths[n] for n in ("fwd", "dq", "dkdv")] == [cuda.PATH_TCGEN05] * 3


@pytest.mark.parametrize("causal", [False, True])
def test_more_work_units_than_sms(causal):
    """160 heads of 512 rows: every persistent CTA walks several units (and, under a causal mask,
    long and short tiles alternately); three heads are checked against the oracle."""
    bh, seq, d = 160, 512, 128
    q, k, v, do = (ref.round_to(t, "bf16") for t in inputs.attention_normal(bh, seq, d, seed=11))
    heads = [0, 77, 159]
    want = tmtest.oracle_attention(q[heads], k[heads], v[heads], do[heads], causal)
    with tmtest.AttentionRun(q, k, v, do, "bf16", causal, (128, 128), cuda.PATH_TCGEN05) as run:
        o, lse = run.forward()
        dq, dk, dv = run.backward()
    for name, got, ref_value in zip(("O", "dQ", "dK", "dV"), (o, dq, dk, dv),
                                    (want[0], want[2], want[3], want[4])):
        assert ref.relative_error(got[heads], ref_value) <= 2e-2, name
    assert np.max(np.abs(lse[heads] - want[1])) <= 2e-2
    # no head was skipped or written twice with something else: every head is finite and non-zero
    for got in (o, dq, dk, dv):
        per_head = np.abs(got.astype(np.float32)).reshape(bh, -1).max(axis=1)
        assert np.all(np.isfinite(per_head)) and np.all(per_head > 0)


def test_tensor_core_paths_leave_rows_outside_the_grid_alone():
    """grid_x covers 3 of 8 row blocks: the other rows of O, dQ, dK, dV keep their sentinel."""
    from triton_metal import kernels
    from triton_metal.buffer import MetalBuffer
    bh, seq, d, blocks = 2, 1024, 128, 3
    q, k, v, do = (ref.round_to(t, "bf16") for t in inputs.attention_normal(bh, seq, d, seed=5))
    dt = ref.storage_dtype("bf16")
    want = tmtest.oracle_attention(q, k, v, do, False)
    scale = kernels.default_scale(d)
    bufs = {n: MetalBuffer.from_numpy(t.astype(dt)) for n, t in (("q", q), ("k", k), ("v", v), ("do", do))}
    sentinel = np.full((bh, seq, d), -7.0, dtype=np.float32).astype(dt)
    for n in ("o", "dq", "dk", "dv"):
        bufs[n] = MetalBuffer.from_numpy(sentinel)
    for n in ("lse", "delta"):
        bufs[n] = MetalBuffer((bh, seq), "float32")
    h = {n: b.tm_handle for n, b in bufs.items()}
    fwd = kernels.AttnFwd("bf16", d, (128, 128), False)
    pre = kernels.AttnBwdPreprocess("bf16", d, 128)
    dq = kernels.AttnBwdDq("bf16", d, (128, 128), False)
    dkdv = kernels.AttnBwdDkdv("bf16", d, (128, 128), False)
    try:
        for kern in (fwd, dq, dkdv):
            kern.set_path(cuda.PATH_TCGEN05)
        # the forward and the preprocess over every row (the backward reads L and Delta of all
        # queries), then dQ and dK/dV over the first `blocks` row blocks only
        fwd(h["q"], h["k"], h["v"], h["o"], h["lse"], scale, bh, seq)
        full_o = bufs["o"].numpy().astype(np.float32).copy()
        pre(h["o"], h["do"], h["delta"], bh, seq)
        bufs["o"].copy_from(sentinel.ctypes.data, sentinel.nbytes)
        for kern, args in ((fwd, (h["q"], h["k"], h["v"], h["o"], h["lse"], scale, bh, seq)),
                           (dq, (h["q"], h["k"], h["v"], h["do"], h["dq"], h["lse"], h["delta"], scale, bh, seq)),
                           (dkdv, (h["q"], h["k"], h["v"], h["do"], h["dk"], h["dv"], h["lse"], h["delta"],
                                   scale, bh, seq))):
            grid, kinds, values = kern.arguments(*args)
            kern.launch((blocks, grid[1], grid[2]), kinds, values)
        rows = blocks * 128
        got = {n: bufs[n].numpy().astype(np.float32).reshape(bh, seq, d) for n in ("o", "dq", "dk", "dv")}
        assert ref.relative_error(full_o, want[0]) <= 2e-2
        assert ref.relative_error(got["o"][:, :rows], want[0][:, :rows]) <= 2e-2
        assert ref.relative_error(got["dq"][:, :rows], want[2][:, :rows]) <= 2e-2
        assert ref.relative_error(got["dk"][:, :rows], want[3][:, :rows]) <= 2e-2
        assert ref.relative_error(got["dv"][:, :rows], want[4][:, :rows]) <= 2e-2
        for n in ("o", "dq", "dk", "dv"):
            assert np.all(got[n][:, rows:] == -7.0), n
    finally:
        for kern in (fwd, pre, dq, dkdv):
            kern.release()
        for b in bufs.values():
            b.free()


def test_seeded_random_shapes_are_correct_and_repeatable():
    """Twenty seeded shapes (both head dimensions, both masks, f16 and bf16, from one tile to
    several units per CTA): three heads against the oracle, every value finite, and a second
    run of every kernel on the same buffers reproduces the first bit for bit (the kernels keep
    no state between launches and use no atomics)."""
    rng = np.random.default_rng(2024)
    for case in range(20):
        d = int(rng.choice([64, 128]))
        causal = bool(rng.integers(0, 2))
        seq = int(rng.choice([128, 129, 255, 257, 384, 512, 640, 777, 1024, 1100, 1536]))
        bh = int(rng.choice([1, 3, 40, 150, 300])) if seq <= 512 else int(rng.choice([1, 2, 5, 37]))
        element = "bf16" if rng.integers(0, 4) else "f16"
        q, k, v, do = (ref.round_to(t, element) for t in inputs.attention_normal(bh, seq, d, seed=case))
        heads = sorted({0, bh // 2, bh - 1})
        want = tmtest.oracle_attention(q[heads], k[heads], v[heads], do[heads], causal)
        with tmtest.AttentionRun(q, k, v, do, element, causal, (128, 128), cuda.PATH_TCGEN05) as run:
            first = run.forward()[:1] + run.backward()
            second = run.forward()[:1] + run.backward()
        label = f"bh{bh} s{seq} d{d} causal={causal} {element}"
        for name, got, again, ref_value in zip(("O", "dQ", "dK", "dV"), first, second,
                                               (want[0], want[2], want[3], want[4])):
            assert ref.relative_error(got[heads], ref_value) <= 2e-2, (label, name)
            assert np.all(np.isfinite(got.astype(np.float32))), (label, name)
            assert np.array_equal(got, again), (label, name)
