"""Helpers shared by the GPU parity tests: move numpy arrays through the C ABI
and run the five kernels the way the reference's drivers do."""

import numpy as np

from oracle import reference_math as ref
from triton_metal import _core, kernels
from triton_metal.buffer import MetalBuffer

BUFFER_DTYPE = {"f32": "float32", "f16": "float16", "bf16": "bfloat16"}


def upload(array, element):
    return MetalBuffer.from_numpy(np.ascontiguousarray(array).astype(ref.storage_dtype(element)))


def put(buffer, array, element="f32"):
    """Overwrite a buffer from a numpy array (kept alive for the whole call)."""
    staged = np.ascontiguousarray(array).astype(ref.storage_dtype(element), copy=False)
    staged = np.ascontiguousarray(staged)
    buffer.copy_from(staged.ctypes.data, staged.nbytes)
    return staged


def empty(shape, element):
    return MetalBuffer(shape, BUFFER_DTYPE[element])


def fetch(buffer):
    return buffer.numpy().astype(np.float32)


def run_matmul(a, b, element, block=(128, 128, 64), path=0, strides=None, c_shape=None,
               c_fill=None, grid=None):
    """C = A @ B through tm_launch.  `a`, `b` are float32 arrays already rounded
    to `element`.  Returns (C as float32, path used)."""
    M, K = a.shape
    N = b.shape[1]
    ab, bb = upload(a, element), upload(b, element)
    cb = empty(c_shape or (M, N), element)
    if c_fill is not None:
        put(cb, np.full(c_shape or (M, N), c_fill, dtype=np.float32), element)
    mm = kernels.Matmul(element, block)
    try:
        mm.set_path(path)
        g, kinds, values = mm.arguments(ab.tm_handle, bb.tm_handle, cb.tm_handle, M, N, K, strides)
        mm.launch(grid or g, kinds, values)
        return fetch(cb), mm.last_path()
    finally:
        mm.release()
        for buf in (ab, bb, cb):
            buf.free()


class AttentionRun:
    """Forward + backward of one attention problem through the ABI."""

    def __init__(self, q, k, v, do, element, causal=False, block=(128, 128), path=0):
        self.bh, self.seq, self.d = q.shape
        self.element, self.causal = element, causal
        self.scale = kernels.default_scale(self.d)
        self.bufs = {"q": upload(q, element), "k": upload(k, element), "v": upload(v, element),
                     "do": upload(do, element)}
        for name in ("o", "dq", "dk", "dv"):
            self.bufs[name] = empty(q.shape, element)
        for name in ("lse", "delta"):
            self.bufs[name] = MetalBuffer((self.bh, self.seq), "float32")
        self.kernels = {
            "fwd": kernels.AttnFwd(element, self.d, block, causal),
            "pre": kernels.AttnBwdPreprocess(element, self.d, block[0]),
            "dq": kernels.AttnBwdDq(element, self.d, block, causal),
            "dkdv": kernels.AttnBwdDkdv(element, self.d, block, causal),
        }
        for kern in self.kernels.values():
            kern.set_path(path)

    def h(self, name):
        return self.bufs[name].tm_handle

    def forward(self):
        self.kernels["fwd"](self.h("q"), self.h("k"), self.h("v"), self.h("o"), self.h("lse"),
                            self.scale, self.bh, self.seq)
        return fetch(self.bufs["o"]), self.bufs["lse"].numpy()

    def backward(self):
        self.kernels["pre"](self.h("o"), self.h("do"), self.h("delta"), self.bh, self.seq)
        self.kernels["dq"](self.h("q"), self.h("k"), self.h("v"), self.h("do"), self.h("dq"),
                           self.h("lse"), self.h("delta"), self.scale, self.bh, self.seq)
        self.kernels["dkdv"](self.h("q"), self.h("k"), self.h("v"), self.h("do"), self.h("dk"),
                             self.h("dv"), self.h("lse"), self.h("delta"), self.scale, self.bh,
                             self.seq)
        return fetch(self.bufs["dq"]), fetch(self.bufs["dk"]), fetch(self.bufs["dv"])

    def paths(self):
        return {name: kern.last_path() for name, kern in self.kernels.items()}

    def close(self):
        for kern in self.kernels.values():
            kern.release()
        for buf in self.bufs.values():
            buf.free()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


def oracle_attention(q, k, v, do, causal):
    scale = kernels.default_scale(q.shape[-1])
    o, weights = ref.attention_forward(q, k, v, scale, causal)
    dq, dk, dv = ref.attention_backward(q, k, v, weights, do, scale)
    return o, ref.logsumexp_log2(q, k, scale, causal), dq, dk, dv


def require_gpu():
    import pytest
    if not _core.is_usable():
        pytest.fail("libtmcuda cannot run on this machine: " + str(_core.unusable_reason()))
