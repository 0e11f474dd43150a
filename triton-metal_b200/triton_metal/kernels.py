"""The hot kernels (and the small kernels of the reference's ABI tests) as callables over
the `tm_*` ABI.

The reference reaches its kernels by handing Triton IR to `tm_emit_msl`
(Sources/TritonMetalBench/{GEMMKernel,AttentionKernel,AttentionBackwardKernel}.swift
generate that IR; python/examples/*.py get it from `@triton.jit`).  libtmcuda
only scans the `tt.func` header and the first `tt.dot`, so the modules built
here are signature-level: header, one `tt.dot` carrying the BLOCK shape, return.
Argument order is the Python order of python/examples/attention_training.py and
python/examples/matmul.py with all six strides present.
"""

import math

from . import _core, cuda, launcher

ELEMENT = {"float32": "f32", "float16": "f16", "bfloat16": "bf16",
           "f32": "f32", "f16": "f16", "bf16": "bf16"}


def matmul_ir(block_m=128, block_n=128, block_k=64, element="f32", fold_unit_strides=False,
              positional_names=False):
    """`fold_unit_strides`: the nine-argument form real Triton emits for a row-major call - it
    specialises integer arguments equal to 1 into constants, so stride_ak, stride_bn and
    stride_cn are not in the signature (Tests/TritonMetalCoreTests/DotFixtures.swift:108-110).
    `positional_names`: %arg0, %arg1, ... as in the Swift generators' output."""
    e = ELEMENT[element]
    names = ["a_ptr", "b_ptr", "c_ptr", "M", "N", "K", "stride_am", "stride_ak", "stride_bk",
             "stride_bn", "stride_cm", "stride_cn"]
    if fold_unit_strides:
        names = [n for n in names if n not in ("stride_ak", "stride_bn", "stride_cn")]
    parts = []
    for i, n in enumerate(names):
        ty = f"!tt.ptr<{e}>" if n.endswith("_ptr") else "i32"
        parts.append(f"%{'arg' + str(i) if positional_names else n}: {ty}")
    return f"""module {{
  tt.func public @matmul_kernel(
      {", ".join(parts)}) {{
    %acc = tt.dot %a, %b, %zero, inputPrecision = tf32 : tensor<{block_m}x{block_k}x{e}> * tensor<{block_k}x{block_n}x{e}> -> tensor<{block_m}x{block_n}xf32>
    tt.return
  }}
}}
"""


def _attn_ir(name, arguments, lhs, rhs, out, element, causal):
    e = ELEMENT[element]
    attributes = " attributes {tm.causal = true}" if causal else ""
    dot = ""
    if rhs is not None:
        dot = (f"    %s = tt.dot %x, %y, %z : tensor<{lhs[0]}x{lhs[1]}x{e}> * "
               f"tensor<{rhs[0]}x{rhs[1]}x{e}> -> tensor<{out[0]}x{out[1]}xf32>\n")
    else:
        dot = f"    %o = tt.load %p : tensor<{lhs[0]}x{lhs[1]}x{e}>\n"
    return (f"module {{\n  tt.func public @{name}({arguments.format(e=e)}){attributes} {{\n"
            f"{dot}    tt.return\n  }}\n}}\n")


def attn_fwd_ir(block_m=128, block_n=128, head_dim=128, element="f32", causal=False, order="python"):
    """`order`: "python" - python/examples/attention_training.py:38 (L fifth, N_CTX last);
    "swift" - Sources/TritonMetalBench/AttentionKernel.swift:75-78 with the row statistic
    (sm_scale fifth, L and stride_lse last); "swift_no_stats" - its eight-argument form."""
    if order == "python":
        args = ("%Q: !tt.ptr<{e}>, %K: !tt.ptr<{e}>, %V: !tt.ptr<{e}>, %O: !tt.ptr<{e}>, "
                "%L: !tt.ptr<f32>, %sm_scale: f32, %stride_head: i32, %stride_seq: i32, "
                "%stride_lse: i32, %N_CTX: i32")
    else:
        args = ("%Q: !tt.ptr<{e}>, %K: !tt.ptr<{e}>, %V: !tt.ptr<{e}>, %O: !tt.ptr<{e}>, "
                "%sm_scale: f32, %stride_head: i32, %stride_seq: i32, %n_ctx: i32")
        if order == "swift":
            args += ", %L: !tt.ptr<f32>, %stride_lse: i32"
    return _attn_ir("attn_fwd", args, (block_m, head_dim), (head_dim, block_n),
                    (block_m, block_n), element, causal)


def attn_bwd_preprocess_ir(block_m=128, head_dim=128, element="f32"):
    args = ("%O: !tt.ptr<{e}>, %DO: !tt.ptr<{e}>, %Delta: !tt.ptr<f32>, %stride_head: i32, "
            "%stride_seq: i32, %stride_lse: i32, %N_CTX: i32")
    return _attn_ir("attn_bwd_preprocess", args, (block_m, head_dim), None, None, element, False)


def attn_bwd_dq_ir(block_m=128, block_n=128, head_dim=128, element="f32", causal=False):
    args = ("%Q: !tt.ptr<{e}>, %K: !tt.ptr<{e}>, %V: !tt.ptr<{e}>, %DO: !tt.ptr<{e}>, "
            "%DQ: !tt.ptr<{e}>, %L: !tt.ptr<f32>, %D: !tt.ptr<f32>, %sm_scale: f32, "
            "%stride_head: i32, %stride_seq: i32, %stride_lse: i32, %N_CTX: i32")
    return _attn_ir("attn_bwd_dq", args, (block_m, head_dim), (head_dim, block_n),
                    (block_m, block_n), element, causal)


def attn_bwd_dkdv_ir(block_m=128, block_n=128, head_dim=128, element="f32", causal=False):
    args = ("%Q: !tt.ptr<{e}>, %K: !tt.ptr<{e}>, %V: !tt.ptr<{e}>, %DO: !tt.ptr<{e}>, "
            "%DK: !tt.ptr<{e}>, %DV: !tt.ptr<{e}>, %L: !tt.ptr<f32>, %D: !tt.ptr<f32>, "
            "%sm_scale: f32, %stride_head: i32, %stride_seq: i32, %stride_lse: i32, %N_CTX: i32")
    return _attn_ir("attn_bwd_dkdv", args, (block_n, head_dim), (head_dim, block_m),
                    (block_n, block_m), element, causal)


# ---- the one-dimensional kernels of the reference's ABI tests -------------------------
# (Tests/TritonMetalCoreTests/Fixtures.swift, python/tests/test_plugin_shape.py).  Full
# programs, not signature stubs: libtmcuda checks that the body holds the operations its
# precompiled kernel of that name performs.

def _masked_index(block, count):
    """pid*BLOCK + arange(BLOCK) and its `< n` mask, as SSA lines."""
    return f"""    %block = arith.constant {block} : i32
    %pid = tt.get_program_id x : i32
    %first = arith.muli %pid, %block : i32
    %lane = tt.make_range {{end = {block} : i32, start = 0 : i32}} : tensor<{block}xi32>
    %firsts = tt.splat %first : i32 -> tensor<{block}xi32>
    %index = arith.addi %firsts, %lane : tensor<{block}xi32>
    %counts = tt.splat {count} : i32 -> tensor<{block}xi32>
    %mask = arith.cmpi slt, %index, %counts : tensor<{block}xi32>
"""


def _load(block, value, pointer):
    return f"""    %{value}_base = tt.splat {pointer} : !tt.ptr<f32> -> tensor<{block}x!tt.ptr<f32>>
    %{value}_ptr = tt.addptr %{value}_base, %index : tensor<{block}x!tt.ptr<f32>>, tensor<{block}xi32>
    %{value} = tt.load %{value}_ptr, %mask : tensor<{block}x!tt.ptr<f32>>
"""


def _store(block, value, pointer):
    return f"""    %out_base = tt.splat {pointer} : !tt.ptr<f32> -> tensor<{block}x!tt.ptr<f32>>
    %out_ptr = tt.addptr %out_base, %index : tensor<{block}x!tt.ptr<f32>>, tensor<{block}xi32>
    tt.store %out_ptr, %{value}, %mask : tensor<{block}x!tt.ptr<f32>>
    tt.return
"""


def elementwise_ir(kind, block):
    """copy: out = in; add / mul: out = a (+|*) b; scale_bias: out = in * scale + bias."""
    if kind == "copy":
        head = "@copy_kernel(%arg0: !tt.ptr<f32>, %arg1: !tt.ptr<f32>, %arg2: i32)"
        body = _masked_index(block, "%arg2") + _load(block, "x", "%arg0") + _store(block, "x", "%arg1")
    elif kind in ("add", "mul"):
        head = (f"@{kind}_kernel(%arg0: !tt.ptr<f32>, %arg1: !tt.ptr<f32>, %arg2: !tt.ptr<f32>, "
                "%arg3: i32)")
        body = (_masked_index(block, "%arg3") + _load(block, "x", "%arg0") + _load(block, "y", "%arg1")
                + f"    %r = arith.{kind}f %x, %y : tensor<{block}xf32>\n" + _store(block, "r", "%arg2"))
    elif kind == "scale_bias":
        head = ("@scale_bias_kernel(%arg0: !tt.ptr<f32>, %arg1: !tt.ptr<f32>, %arg2: f32, %arg3: f32, "
                "%arg4: i32)")
        body = (_masked_index(block, "%arg4") + _load(block, "x", "%arg0")
                + f"    %scales = tt.splat %arg2 : f32 -> tensor<{block}xf32>\n"
                + f"    %scaled = arith.mulf %x, %scales : tensor<{block}xf32>\n"
                + f"    %biases = tt.splat %arg3 : f32 -> tensor<{block}xf32>\n"
                + f"    %r = arith.addf %scaled, %biases : tensor<{block}xf32>\n" + _store(block, "r", "%arg1"))
    else:
        raise ValueError(f"unknown element-wise kernel '{kind}'")
    return f"module {{\n  tt.func public {head} {{\n{body}  }}\n}}\n"


def softmax_ir(block):
    """One program per row: exp(x - max) / sum over the first n_cols (< BLOCK) columns."""
    t = f"tensor<{block}xf32>"
    return f"""module {{
  tt.func public @softmax_kernel(%arg0: !tt.ptr<f32>, %arg1: !tt.ptr<f32>, %arg2: i32, %arg3: i32, %arg4: i32) {{
    %minus_inf = arith.constant dense<0xFF800000> : {t}
    %row = tt.get_program_id x : i32
    %in_off = arith.muli %row, %arg2 : i32
    %in_row = tt.addptr %arg0, %in_off : !tt.ptr<f32>, i32
    %col = tt.make_range {{end = {block} : i32, start = 0 : i32}} : tensor<{block}xi32>
    %in_base = tt.splat %in_row : !tt.ptr<f32> -> tensor<{block}x!tt.ptr<f32>>
    %in_ptr = tt.addptr %in_base, %col : tensor<{block}x!tt.ptr<f32>>, tensor<{block}xi32>
    %ncols = tt.splat %arg4 : i32 -> tensor<{block}xi32>
    %mask = arith.cmpi slt, %col, %ncols : tensor<{block}xi32>
    %x = tt.load %in_ptr, %mask, %minus_inf : {t}
    %max = "tt.reduce"(%x) <{{axis = 0 : i32}}> ({{
    ^bb0(%a: f32, %b: f32):
      %m = arith.maxnumf %a, %b : f32
      tt.reduce.return %m : f32
    }}) : ({t}) -> f32
    %maxes = tt.splat %max : f32 -> {t}
    %shifted = arith.subf %x, %maxes : {t}
    %e = math.exp %shifted : {t}
    %sum = "tt.reduce"(%e) <{{axis = 0 : i32}}> ({{
    ^bb0(%c: f32, %d: f32):
      %s = arith.addf %c, %d : f32
      tt.reduce.return %s : f32
    }}) : ({t}) -> f32
    %sums = tt.splat %sum : f32 -> {t}
    %y = arith.divf %e, %sums : {t}
    %out_off = arith.muli %row, %arg3 : i32
    %out_row = tt.addptr %arg1, %out_off : !tt.ptr<f32>, i32
    %out_base = tt.splat %out_row : !tt.ptr<f32> -> tensor<{block}x!tt.ptr<f32>>
    %out_ptr = tt.addptr %out_base, %col : tensor<{block}x!tt.ptr<f32>>, tensor<{block}xi32>
    tt.store %out_ptr, %y, %mask : tensor<{block}x!tt.ptr<f32>>
    tt.return
  }}
}}
"""


def sae_encode_ir(block_m=64, block_f=64, block_d=16):
    """out = relu(x @ w + bias), fp32, row-major (Sources/TritonMetalMLX/SAEEncoder.swift:40-200).
    Signature-level like the matmul: the header, the tt.dot that carries the BLOCK shape and the
    epilogue operations libtmcuda checks for (+ bias, maximum with 0, store)."""
    t = f"tensor<{block_m}x{block_f}xf32>"
    return f"""module {{
  tt.func public @sae_encode_kernel(
      %x: !tt.ptr<f32>, %w: !tt.ptr<f32>, %bias: !tt.ptr<f32>, %out: !tt.ptr<f32>,
      %M: i32, %D: i32, %F: i32) {{
    %acc = tt.dot %xv, %wv, %zero, inputPrecision = tf32 : tensor<{block_m}x{block_d}xf32> * tensor<{block_d}x{block_f}xf32> -> {t}
    %biased = arith.addf %acc, %b_bcast : {t}
    %activated = arith.maximumf %biased, %relu0 : {t}
    tt.store %o_ptrs, %activated, %o_mask : tensor<{block_m}x{block_f}x!tt.ptr<f32>>
    tt.return
  }}
}}
"""


class _Handle:
    """A bare buffer handle presented the way the launcher takes pointer arguments."""
    __slots__ = ("tm_handle",)

    def __init__(self, handle):
        self.tm_handle = handle


class Kernel:
    """IR -> metadata + descriptor -> library -> pipeline, the flow of MetalBackend.make_msl and
    MetalUtils.load_binary (python/plugin/backend/compiler.py:131-146, driver.py:31-40), and
    launches marshalled by MetalLauncher's rules (driver.py:58-92) from the `metal_args` that
    `tm_kernel_info` reports - no per-kernel list of argument kinds is written down here.
    `release()` drops both handles."""

    def __init__(self, ir, name, num_warps=4, signature=None):
        self.name = name
        self.threads = 32 * num_warps
        self.metadata, image = launcher.make_msl(ir, num_warps)
        self.descriptor = image.decode("utf-8")
        self.metal_args = self.metadata["metal_args"]
        if signature is None:       # every parameter of the Python definition is in the IR
            signature = {f"arg{i}": "runtime" for i in range(len(self.metal_args))}
        self.launcher = launcher.Launcher(signature)
        self.library, self.handle, _, _, _ = launcher.load_binary(name, image)

    def marshal(self, *call_args):
        """(kinds, values) for the arguments of a Python-level call; integers in pointer
        positions are buffer handles."""
        call_args = list(call_args)
        for index, kind, _dtype in self.metal_args:
            pos = self.launcher.positions[index]
            if kind == "pointer" and isinstance(call_args[pos], int):
                call_args[pos] = _Handle(call_args[pos])
        return self.launcher.marshal(self.metal_args, call_args)

    def set_path(self, path):
        cuda.set_option(self.handle, "path", path)

    def set_causal(self, causal):
        cuda.set_option(self.handle, "causal", int(bool(causal)))

    def last_path(self):
        return cuda.last_path(self.handle)

    def launch(self, grid, kinds, values):
        _core.launch(self.handle, grid, self.threads, kinds, values)

    def launch_async(self, grid, kinds, values):
        cuda.launch_async(self.handle, grid, self.threads, kinds, values)

    def time(self, grid, kinds, values, repeats):
        return cuda.launch_timed(self.handle, grid, self.threads, kinds, values, repeats)

    def release(self):
        if self.handle:
            _core.release_kernel(self.handle)
            _core.release_library(self.library)
            self.handle = self.library = 0


def cdiv(a, b):
    return (a + b - 1) // b


class Matmul(Kernel):
    """`matmul_kernel`: C[M,N] = A[M,K] @ B[K,N], fp32 accumulate."""

    def __init__(self, element="f32", block=(128, 128, 64), num_warps=4):
        self.block = block
        super().__init__(matmul_ir(*block, element=element), "matmul_kernel", num_warps)

    def arguments(self, a, b, c, M, N, K, strides=None):
        if strides is None:
            strides = (K, 1, N, 1, N, 1)
        kinds, values = self.marshal(a, b, c, M, N, K, *strides)
        grid = (cdiv(M, self.block[0]), cdiv(N, self.block[1]), 1)
        return grid, kinds, values

    def __call__(self, a, b, c, M, N, K, strides=None):
        self.launch(*self.arguments(a, b, c, M, N, K, strides))


class AttnFwd(Kernel):
    def __init__(self, element="f32", head_dim=128, block=(128, 128), causal=False, num_warps=4):
        self.block, self.head_dim = block, head_dim
        super().__init__(attn_fwd_ir(block[0], block[1], head_dim, element, causal), "attn_fwd",
                         num_warps)

    def arguments(self, q, k, v, o, lse, scale, bh, seq):
        d = self.head_dim
        kinds, values = self.marshal(q, k, v, o, lse, scale, seq * d, d, seq, seq)
        return (cdiv(seq, self.block[0]), bh, 1), kinds, values

    def __call__(self, *args):
        self.launch(*self.arguments(*args))


class AttnBwdPreprocess(Kernel):
    def __init__(self, element="f32", head_dim=128, block_m=128, num_warps=4):
        self.block_m, self.head_dim = block_m, head_dim
        super().__init__(attn_bwd_preprocess_ir(block_m, head_dim, element),
                         "attn_bwd_preprocess", num_warps)

    def arguments(self, o, do, delta, bh, seq):
        d = self.head_dim
        kinds, values = self.marshal(o, do, delta, seq * d, d, seq, seq)
        return (cdiv(seq, self.block_m), bh, 1), kinds, values

    def __call__(self, *args):
        self.launch(*self.arguments(*args))


class AttnBwdDq(Kernel):
    def __init__(self, element="f32", head_dim=128, block=(128, 128), causal=False, num_warps=4):
        self.block, self.head_dim = block, head_dim
        super().__init__(attn_bwd_dq_ir(block[0], block[1], head_dim, element, causal),
                         "attn_bwd_dq", num_warps)

    def arguments(self, q, k, v, do, dq, lse, delta, scale, bh, seq):
        d = self.head_dim
        kinds, values = self.marshal(q, k, v, do, dq, lse, delta, scale, seq * d, d, seq, seq)
        return (cdiv(seq, self.block[0]), bh, 1), kinds, values

    def __call__(self, *args):
        self.launch(*self.arguments(*args))


class AttnBwdDkdv(Kernel):
    def __init__(self, element="f32", head_dim=128, block=(128, 128), causal=False, num_warps=4):
        self.block, self.head_dim = block, head_dim
        super().__init__(attn_bwd_dkdv_ir(block[0], block[1], head_dim, element, causal),
                         "attn_bwd_dkdv", num_warps)

    def arguments(self, q, k, v, do, dk, dv, lse, delta, scale, bh, seq):
        d = self.head_dim
        kinds, values = self.marshal(q, k, v, do, dk, dv, lse, delta, scale, seq * d, d, seq, seq)
        return (cdiv(seq, self.block[1]), bh, 1), kinds, values

    def __call__(self, *args):
        self.launch(*self.arguments(*args))


class SaeEncode(Kernel):
    """out[M, F] = relu(x[M, D] @ w[D, F] + bias[F]); grid (cdiv(M, BM), cdiv(F, BF))."""

    def __init__(self, block=(64, 64, 16), num_warps=4):
        super().__init__(sae_encode_ir(*block), "sae_encode_kernel", num_warps)
        self.block = block

    def arguments(self, x, w, bias, out, rows, model, features):
        grid = (cdiv(rows, self.block[0]), cdiv(features, self.block[1]), 1)
        kinds, values = self.marshal(x, w, bias, out, rows, model, features)
        return grid, kinds, values

    def __call__(self, *a):
        self.launch(*self.arguments(*a))


class Elementwise(Kernel):
    """copy / add / mul / scale_bias over n fp32 elements, BLOCK per program."""

    NAMES = {"copy": "copy_kernel", "add": "add_kernel", "mul": "mul_kernel",
             "scale_bias": "scale_bias_kernel"}

    def __init__(self, kind, block=1024, num_warps=4):
        super().__init__(elementwise_ir(kind, block), self.NAMES[kind], num_warps)
        self.kind, self.block = kind, block

    def arguments(self, *operands, n, scale=1.0, bias=0.0, programs=None):
        """operands: buffer handles (in, out) or (a, b, out)."""
        grid = (programs if programs is not None else max(1, cdiv(n, self.block)), 1, 1)
        if self.kind == "scale_bias":
            kinds, values = self.marshal(operands[0], operands[1], scale, bias, n)
        else:
            kinds, values = self.marshal(*operands, n)
        return grid, kinds, values

    def __call__(self, *operands, **kw):
        self.launch(*self.arguments(*operands, **kw))


class Softmax(Kernel):
    """Row softmax, one program per row, n_cols <= BLOCK columns."""

    def __init__(self, block=128, num_warps=4):
        super().__init__(softmax_ir(block), "softmax_kernel", num_warps)
        self.block = block

    def arguments(self, x, y, rows, n_cols, stride_in=None, stride_out=None):
        stride_in = n_cols if stride_in is None else stride_in
        stride_out = n_cols if stride_out is None else stride_out
        kinds, values = self.marshal(x, y, stride_in, stride_out, n_cols)
        return (rows, 1, 1), kinds, values

    def __call__(self, *a, **kw):
        self.launch(*self.arguments(*a, **kw))


def default_scale(head_dim):
    return 1.0 / math.sqrt(head_dim)
