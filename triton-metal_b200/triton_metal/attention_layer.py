"""One attention layer with Q/K/V/O projections, trained by SGD, with every step on libtmcuda.

This is the small fp32 training configuration: X [seq, d_model] is projected by Wq, Wk, Wv,
split into heads, run through `attn_fwd`, merged, projected by Wo and compared with a target
(mean squared error); the backward pass runs `attn_bwd_preprocess`, `attn_bwd_dq` and
`attn_bwd_dkdv` and the transposed projections, and the update is plain SGD.  The reference's
example (python/examples/attention_training.py:255-330) trains q, k and v directly and keeps
the attention on the GPU and everything else in numpy; here the eight matrix products of a
step go through `matmul_kernel` as well - transposes are expressed with its stride arguments,
the head split with the attention kernels' `stride_head` / `stride_seq`, so no tensor is
reshuffled on the host - and the element-wise pieces (Y - T, the 2/n factor, W - lr*G) through
`scale_bias_kernel` and `add_kernel`.  Only the scalar loss is reduced on the host, from a
read-back of Y - T.
"""

import numpy as np

from . import kernels
from .buffer import MetalBuffer


class ProjectionAttention:
    def __init__(self, x, target, weights, heads, attn_block=(16, 32), matmul_block=(32, 32, 32)):
        self.seq, self.d_model = x.shape
        self.heads, self.dh = heads, self.d_model // heads
        self.scale = kernels.default_scale(self.dh)
        S, dm = self.seq, self.d_model
        f32 = "float32"
        self.buf = {"x": MetalBuffer.from_numpy(np.ascontiguousarray(x, dtype=np.float32)),
                    "target": MetalBuffer.from_numpy(np.ascontiguousarray(target, dtype=np.float32))}
        for name, w in zip(("wq", "wk", "wv", "wo"), weights):
            self.buf[name] = MetalBuffer.from_numpy(np.ascontiguousarray(w, dtype=np.float32))
            self.buf["d" + name] = MetalBuffer((dm, dm), f32)
            self.buf["step_" + name] = MetalBuffer((dm, dm), f32)
        for name in ("q", "k", "v", "o", "y", "diff", "neg_target", "dy", "do", "dq", "dk", "dv"):
            self.buf[name] = MetalBuffer((S, dm), f32)
        for name in ("lse", "delta"):
            self.buf[name] = MetalBuffer((heads, S), f32)
        self.mm = kernels.Matmul("f32", matmul_block)
        self.fwd = kernels.AttnFwd("f32", self.dh, attn_block)
        self.pre = kernels.AttnBwdPreprocess("f32", self.dh, attn_block[0])
        self.dq = kernels.AttnBwdDq("f32", self.dh, attn_block)
        self.dkdv = kernels.AttnBwdDkdv("f32", self.dh, attn_block)
        self.add = kernels.Elementwise("add", 1024)
        self.axpb = kernels.Elementwise("scale_bias", 1024)
        self.attn_block = attn_block
        # -T once: Y - T is then one add_kernel launch per step
        self._scale("target", "neg_target", -1.0, S * dm)

    def h(self, name):
        return self.buf[name].tm_handle

    # ---- launches ---------------------------------------------------------------------
    def _matmul(self, a, b, c, M, N, K, a_transposed=False, b_transposed=False):
        """c[M,N] = op(a) @ op(b) with row-major storage; a transposed operand is the same
        buffer read with its two strides exchanged."""
        sam, sak = (1, M) if a_transposed else (K, 1)
        sbk, sbn = (1, K) if b_transposed else (N, 1)
        self.mm(self.h(a), self.h(b), self.h(c), M, N, K, strides=(sam, sak, sbk, sbn, N, 1))

    def _scale(self, src, dst, factor, n):
        self.axpb(self.h(src), self.h(dst), n=n, scale=factor, bias=0.0)

    def _add(self, a, b, dst, n):
        self.add(self.h(a), self.h(b), self.h(dst), n=n)

    def _attention_strides(self):
        # head h of a [seq, d_model] tensor: rows d_model apart, heads dh columns apart
        return self.dh, self.d_model, self.seq, self.seq     # stride_head, stride_seq, stride_lse, n_ctx

    # ---- one training step ------------------------------------------------------------
    def forward(self):
        """Runs the layer; returns the loss mean((Y - T)^2)."""
        S, dm, H = self.seq, self.d_model, self.heads
        for w, out in (("wq", "q"), ("wk", "k"), ("wv", "v")):
            self._matmul("x", w, out, S, dm, dm)
        sh, ss, sl, n = self._attention_strides()
        kinds, values = self.fwd.marshal(self.h("q"), self.h("k"), self.h("v"), self.h("o"),
                                         self.h("lse"), self.scale, sh, ss, sl, n)
        self.fwd.launch((kernels.cdiv(S, self.attn_block[0]), H, 1), kinds, values)
        self._matmul("o", "wo", "y", S, dm, dm)
        self._add("y", "neg_target", "diff", S * dm)
        diff = self.buf["diff"].numpy()
        return float(np.mean(diff.astype(np.float64) ** 2))

    def backward(self):
        """Gradients of the loss with respect to the four weight matrices (left in dw*)."""
        S, dm, H = self.seq, self.d_model, self.heads
        self._scale("diff", "dy", 2.0 / (S * dm), S * dm)
        self._matmul("o", "dy", "dwo", dm, dm, S, a_transposed=True)           # merged^T dY
        self._matmul("dy", "wo", "do", S, dm, dm, b_transposed=True)           # dY Wo^T
        sh, ss, sl, n = self._attention_strides()
        grid_m = (kernels.cdiv(S, self.attn_block[0]), H, 1)
        grid_n = (kernels.cdiv(S, self.attn_block[1]), H, 1)
        k, v = self.pre.marshal(self.h("o"), self.h("do"), self.h("delta"), sh, ss, sl, n)
        self.pre.launch(grid_m, k, v)
        k, v = self.dq.marshal(self.h("q"), self.h("k"), self.h("v"), self.h("do"), self.h("dq"),
                               self.h("lse"), self.h("delta"), self.scale, sh, ss, sl, n)
        self.dq.launch(grid_m, k, v)
        k, v = self.dkdv.marshal(self.h("q"), self.h("k"), self.h("v"), self.h("do"), self.h("dk"),
                                 self.h("dv"), self.h("lse"), self.h("delta"), self.scale, sh, ss, sl, n)
        self.dkdv.launch(grid_n, k, v)
        for grad, out in (("dq", "dwq"), ("dk", "dwk"), ("dv", "dwv")):
            self._matmul("x", grad, out, dm, dm, S, a_transposed=True)         # X^T dQ
        return tuple(self.buf[n].numpy() for n in ("dwq", "dwk", "dwv", "dwo"))

    def sgd(self, lr):
        n = self.d_model * self.d_model
        for w in ("wq", "wk", "wv", "wo"):
            self._scale("d" + w, "step_" + w, -lr, n)
            self._add(w, "step_" + w, w, n)

    def weights(self):
        return tuple(self.buf[n].numpy() for n in ("wq", "wk", "wv", "wo"))

    def close(self):
        for kern in (self.mm, self.fwd, self.pre, self.dq, self.dkdv, self.add, self.axpb):
            kern.release()
        for buf in self.buf.values():
            buf.free()
