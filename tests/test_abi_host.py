"""The C-ABI boundary without a GPU: the library loads, exports every symbol
include/tm.h declares, and reproduces the reference's error behaviour
(Tests/TritonMetalCoreTests/CABITests.swift, python/tests/test_plugin_shape.py).
No compute call is made here."""

import ctypes
import json
import os
import re
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
HEADER = ROOT / "include" / "tm.h"
# the reference checkout, when one is at hand (tests that need it skip otherwise)
REFERENCE = Path(os.environ.get("TRITON_METAL_REFERENCE") or "/nonexistent-reference-checkout")

from triton_metal import _core, kernels  # noqa: E402


def declared_symbols():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(tmx?_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_23_reference_exports():
    names = [n for n in declared_symbols() if n.startswith("tm_")]
    assert sorted(names) == sorted(_core.EXPORTS), set(names) ^ set(_core.EXPORTS)
    assert len(names) == 23


def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(_core.library_path())
    for name in declared_symbols():
        assert getattr(lib, name) is not None, name


def test_version_and_error_slot(core):
    assert core.version() == "0.0.1"
    assert core.last_error() == "no error"
    with pytest.raises(RuntimeError, match="is not live"):
        core.buffer_length(999_999)
    assert core.last_error() == "no error"      # reading the error cleared it


def test_parse_and_unsupported_op_errors(core):
    with pytest.raises(RuntimeError, match="no tt.func"):
        core.emit_msl("module {}")
    with pytest.raises(RuntimeError, match="no tt.func"):
        core.kernel_info("module {}")
    ir = """
    module {
      tt.func public @k(%arg0: !tt.ptr<f32>) {
        %0 = tt.histogram %arg0 : !tt.ptr<f32>
        tt.return
      }
    }
    """
    with pytest.raises(RuntimeError, match=r"unsupported op 'tt.histogram'"):
        core.emit_msl(ir)


def test_other_kernels_are_refused_by_name(core):
    ir = "module {\n  tt.func public @iadd_kernel(%a: !tt.ptr<i32>, %n: i32) {\n    tt.return\n  }\n}"
    with pytest.raises(RuntimeError, match="kernel 'iadd_kernel'.*no sm_100a implementation"):
        core.emit_msl(ir)


def test_one_dimensional_kernels_scan(core):
    """kernel_info of the kernels the reference's ABI tests launch: name, BLOCK from
    tt.make_range, threads = 32 * num_warps (CABITests.swift:49-56,
    test_plugin_shape.py:148-155, :228)."""
    cases = [("copy", 256, "copy_kernel", ["pointer", "pointer", "scalar"]),
             ("add", 1024, "add_kernel", ["pointer"] * 3 + ["scalar"]),
             ("mul", 128, "mul_kernel", ["pointer"] * 3 + ["scalar"]),
             ("scale_bias", 64, "scale_bias_kernel", ["pointer", "pointer", "scalar", "scalar", "scalar"])]
    for kind, block, name, arg_kinds in cases:
        info = json.loads(core.kernel_info(kernels.elementwise_ir(kind, block), 4))["kernels"][0]
        assert (info["name"], info["block_size"], info["block_shape"]) == (name, block, [block])
        assert info["threads_per_threadgroup"] == 128
        assert [a["kind"] for a in info["args"]] == arg_kinds
    info = json.loads(core.kernel_info(kernels.elementwise_ir("scale_bias", 64), 4))["kernels"][0]
    assert [a["dtype"] for a in info["args"]] == ["f32", "f32", "f32", "f32", "i32"]
    info = json.loads(core.kernel_info(kernels.softmax_ir(128), 2))["kernels"][0]
    assert (info["name"], info["block_size"], info["threads_per_threadgroup"]) == ("softmax_kernel", 128, 64)


def test_sae_encoder_scans(core):
    """sae_encode_kernel(x, w, bias, out, M, D, F): block shape from its tt.dot
    (Sources/TritonMetalMLX/SAEEncoder.swift:40-56)."""
    info = json.loads(core.kernel_info(kernels.sae_encode_ir(64, 32, 16), 8))["kernels"][0]
    assert (info["name"], info["block_shape"], info["block_size"]) == ("sae_encode_kernel", [64, 32], 2048)
    assert info["threads_per_threadgroup"] == 256
    assert [a["kind"] for a in info["args"]] == ["pointer"] * 4 + ["scalar"] * 3
    with pytest.raises(RuntimeError, match="body of 'sae_encode_kernel'"):
        core.emit_msl(kernels.sae_encode_ir().replace("arith.maximumf", "arith.minimumf"))
    with pytest.raises(RuntimeError, match="f32 only"):
        core.emit_msl(kernels.sae_encode_ir().replace("f32", "f16"))


def test_a_same_named_kernel_with_another_body_is_refused(core):
    """The precompiled kernels are selected by name; a body that computes something else
    must not be replaced silently."""
    ir = kernels.elementwise_ir("add", 1024).replace("arith.addf", "arith.subf")
    with pytest.raises(RuntimeError, match="body of 'add_kernel'"):
        core.emit_msl(ir)
    with pytest.raises(RuntimeError, match="takes 4 arguments"):
        core.emit_msl(kernels.elementwise_ir("add", 1024).replace(", %arg3: i32", ""))
    with pytest.raises(RuntimeError, match="f32 only"):
        core.emit_msl(kernels.elementwise_ir("copy", 256).replace("f32", "bf16"))


def test_f64_arguments_are_refused(core):
    ir = kernels.matmul_ir().replace("%M: i32", "%M: f64")
    with pytest.raises(RuntimeError, match="f64"):
        core.emit_msl(ir)


def test_null_arguments(core):
    lib = core._lib
    assert not lib.tm_emit_msl(None, 4)
    assert "tm_emit_msl received a NULL module" in core.last_error()
    assert not lib.tm_kernel_info(None, 4)
    assert "tm_kernel_info received a NULL module" in core.last_error()
    assert lib.tm_compile_msl(None) == 0
    assert "tm_compile_msl received NULL source" in core.last_error()
    assert lib.tm_load_kernel(1, None) == 0
    assert "NULL kernel name" in core.last_error()
    assert lib.tm_load_metallib(None, 0) == 0
    assert "empty image" in core.last_error()


def test_invalid_handles(core):
    lib = core._lib
    assert lib.tm_load_kernel(999_999, b"k") == 0
    assert "library handle 999999 is not live" in core.last_error()
    assert lib.tm_buffer_length(999_999) == -1
    assert "is not live" in core.last_error()
    assert lib.tm_free_buffer(999_999) == -1
    assert lib.tm_launch(999_999, 1, 1, 1, 32, None, None, 0) == -1
    assert "kernel handle" in core.last_error()
    assert lib.tm_kernel_max_threads(999_999) == -1
    assert "kernel handle 999999 is not live" in core.last_error()
    assert not lib.tm_buffer_contents(999_999)
    assert "is not live" in core.last_error()
    assert lib.tm_release_kernel(999_999) == -1
    assert lib.tm_release_library(999_999) == -1


def test_compile_errors_give_a_zero_handle(core):
    assert core._lib.tm_compile_msl(b"not msl at all") == 0
    assert "MSL compilation failed" in core.last_error()
    garbage = bytes(range(64))
    assert core._lib.tm_load_metallib(garbage, 64) == 0
    assert "could not load metallib" in core.last_error()


def test_invalid_allocation_and_copy_bounds(core):
    assert core._lib.tm_alloc_buffer(0) == 0
    assert "buffer length must be positive" in core.last_error()
    value = ctypes.c_float(0)
    # NULL / negative bounds are refused before the handle is looked at
    assert core._lib.tm_buffer_write(12345, 0, None, 4) == -1
    assert "invalid bounds" in core.last_error()
    assert core._lib.tm_buffer_write(12345, 0, ctypes.byref(value), -1) == -1
    assert core._lib.tm_buffer_read(12345, -4, ctypes.byref(value), 4) == -1
    assert "invalid bounds" in core.last_error()


def test_library_and_kernel_handles(core, no_leaks):
    descriptor = core.emit_msl(kernels.matmul_ir(64, 64, 16, "bf16"), 8)
    library = core.compile_msl(descriptor)
    image = core.load_metallib(descriptor.encode())
    assert library >= 1 and image == library + 1
    with pytest.raises(RuntimeError, match=r"kernel 'nope' not found in library \(available: matmul_kernel\)"):
        core.load_kernel(library, "nope")
    kernel = core.load_kernel(library, "matmul_kernel")
    assert core.kernel_max_threads(kernel) >= 128
    # typed lookup: a kernel handle is not a library
    with pytest.raises(RuntimeError, match=f"handle {kernel} is not a library"):
        core.load_kernel(kernel, "matmul_kernel")
    # launch argument validation happens before any device work
    kinds = (ctypes.c_int32 * 12)(*([0, 0, 0] + [1] * 8 + [7]))
    values = (ctypes.c_int64 * 12)(*([0] * 12))
    assert core._lib.tm_launch(kernel, 1, 1, 1, 128, kinds, values, 12) == -1
    assert "unknown launch argument kind 7 at position 11" in core.last_error()
    assert core._lib.tm_launch(kernel, 1, 1, 1, 128, None, None, 5) == -1
    assert "NULL argument arrays" in core.last_error()
    kinds = (ctypes.c_int32 * 3)(1, 1, 1)
    assert core._lib.tm_launch(kernel, 1, 1, 1, 128, kinds, values, 3) == -1
    assert "takes 12 arguments" in core.last_error()
    core.release_kernel(kernel)
    core.release_library(image)
    core.release_library(library)
    with pytest.raises(RuntimeError):
        core.release_library(library)


def test_kernel_info_shape(core):
    info = json.loads(core.kernel_info(kernels.attn_fwd_ir(32, 64, 128, "bf16"), 4))
    kernel = info["kernels"][0]
    assert kernel["name"] == "attn_fwd"
    assert kernel["block_shape"] == [32, 64] and kernel["block_size"] == 32 * 64
    assert kernel["threads_per_threadgroup"] == 128
    assert [a["kind"] for a in kernel["args"]] == ["pointer"] * 5 + ["scalar"] * 5
    assert [a["dtype"] for a in kernel["args"]] == ["bf16"] * 4 + ["f32", "f32"] + ["i32"] * 4
    assert [a["index"] for a in kernel["args"]] == list(range(10))


def test_argument_orders_of_both_reference_front_ends(core):
    """The Swift fixture puts sm_scale at position 4 and L at the end
    (AttentionKernel.swift:75-78); the Python kernel puts L at 4
    (attention_training.py:38).  Both must scan, by name or by position."""
    swift = """module {
      tt.func public @attn_fwd(
          %Q: !tt.ptr<f16>, %K: !tt.ptr<f16>, %V: !tt.ptr<f16>,
          %O: !tt.ptr<f16>, %sm_scale: f32,
          %stride_head: i32, %stride_seq: i32, %n_ctx: i32,
          %L: !tt.ptr<f32>, %stride_lse: i32) {
        tt.return
      }
    }"""
    text = core.emit_msl(swift)
    roles = [line.split()[4] for line in text.splitlines() if line.strip().startswith("arg ")]
    positional = swift.replace("%Q", "%arg0").replace("%K:", "%arg1:").replace("%V", "%arg2") \
        .replace("%O", "%arg3").replace("%sm_scale", "%arg4").replace("%stride_head", "%arg5") \
        .replace("%stride_seq", "%arg6").replace("%n_ctx", "%arg7").replace("%L", "%arg8") \
        .replace("%stride_lse", "%arg9")
    text2 = core.emit_msl(positional)
    roles2 = [line.split()[4] for line in text2.splitlines() if line.strip().startswith("arg ")]
    assert roles == roles2
    python_order = core.emit_msl(kernels.attn_fwd_ir(16, 32, 64, "f32"))
    roles3 = [line.split()[4] for line in python_order.splitlines() if line.strip().startswith("arg ")]
    assert sorted(roles3) == sorted(roles) and roles3 != roles


def test_matmul_with_unit_strides_folded(core):
    """Real Triton drops the unit-stride arguments (DotFixtures.swift:108-110)."""
    ir = """module {
      tt.func public @matmul_kernel(%a_ptr: !tt.ptr<f32>, %b_ptr: !tt.ptr<f32>,
                                    %c_ptr: !tt.ptr<f32>, %M: i32, %N: i32, %K: i32,
                                    %stride_am: i32, %stride_bk: i32, %stride_cm: i32) {
        tt.return
      }
    }"""
    info = json.loads(core.kernel_info(ir))
    assert len(info["kernels"][0]["args"]) == 9


def test_descriptor_round_trip_keeps_the_causal_attribute(core, no_leaks):
    descriptor = core.emit_msl(kernels.attn_bwd_dq_ir(64, 64, 64, "bf16", causal=True))
    assert "causal 1" in descriptor
    library = core.compile_msl(descriptor)
    kernel = core.load_kernel(library, "attn_bwd_dq")
    core.release_kernel(kernel)
    core.release_library(library)


@pytest.mark.skipif(not REFERENCE.exists(), reason="set TRITON_METAL_REFERENCE to a reference checkout")
def test_reference_generators_scan():
    """The IR text of the reference's own generators (read as text, template
    holes filled here) goes through the scanner."""
    source = (REFERENCE / "Sources/TritonMetalBench/GEMMKernel.swift").read_text()
    body = source.split('return """', 1)[1].split('"""', 1)[0]
    body = body.replace("\\(blockM)", "64").replace("\\(blockN)", "32").replace("\\(blockK)", "16")
    body = body.replace("\\(blockK - 1)", "15").replace("\\(element)", "f32")
    body = body.replace("\\(seed)", "0.000000e+00")
    body = body.replace("\\(store)", "      %52 = arith.mulf %51, %cone : tensor<64x32xf32>")
    body = re.sub(r"\\\n\s*", "", body)
    info = json.loads(_core.kernel_info(body, 8))["kernels"][0]
    assert info["name"] == "matmul_kernel" and info["block_shape"] == [64, 32]
    assert len(info["args"]) == 12
    assert "block_k 16" in _core.emit_msl(body)


@pytest.mark.skipif(not REFERENCE.exists(), reason="set TRITON_METAL_REFERENCE to a reference checkout")
def test_reference_shim_binds_unchanged():
    """python/triton_metal/_core.py of the reference binds all 23 names at import;
    pointed at libtmcuda through its own environment variable it must load."""
    env = dict(os.environ, TRITON_METAL_CORE_LIB=_core.library_path(),
               PYTHONPATH=str(REFERENCE / "python"))
    code = ("from triton_metal import _core; from triton_metal.buffer import MetalBuffer;"
            "assert _core.version() == '0.0.1'; print(_core.live_handle_count())")
    out = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True,
                         cwd="/tmp")
    assert out.returncode == 0, out.stderr
    assert out.stdout.strip() == "0"


def test_descriptors_that_did_not_come_from_emit_are_refused(core):
    """tm_compile_msl / tm_load_metallib re-run the scanner's checks on the descriptor they are
    given: a truncated, stale or edited one is an error, not a kernel that later dereferences
    a buffer it never received."""
    good = core.emit_msl(kernels.matmul_ir(64, 64, 32, "f32"))
    lines = good.splitlines()
    arg_lines = [i for i, l in enumerate(lines) if l.strip().startswith("arg ")]
    # the C pointer is gone (and the later arguments renumbered): a required role is missing
    cut = [l for i, l in enumerate(lines) if i != arg_lines[2]]
    renumbered, n = [], 0
    for l in cut:
        if l.strip().startswith("arg "):
            parts = l.split()
            parts[1] = str(n)
            n += 1
            l = "  " + " ".join(parts)
        renumbered.append(l)
    with pytest.raises(RuntimeError, match="missing a required argument"):
        core.compile_msl("\n".join(renumbered) + "\n")
    # a pointer turned into a scalar
    edited = good.replace(lines[arg_lines[0]], lines[arg_lines[0]].replace("pointer", "scalar"))
    with pytest.raises(RuntimeError, match="should be a pointer"):
        core.compile_msl(edited)
    # truncated before `end`
    with pytest.raises(RuntimeError, match="no complete kernel"):
        core.compile_msl("\n".join(lines[:arg_lines[1]]) + "\n")
    # the one-dimensional kernels and the fused encoder exist for f32 only
    sae = core.emit_msl(kernels.sae_encode_ir())
    with pytest.raises(RuntimeError, match="f32 only|mixes element types"):
        core.compile_msl(sae.replace("element f32", "element bf16"))
    with pytest.raises(RuntimeError, match="not a tmcuda kernel descriptor"):
        core.load_metallib(cut[2].encode())
    with pytest.raises(RuntimeError, match="could not load metallib"):
        core.load_metallib(("\n".join(renumbered) + "\n").encode())
    assert core.last_error() == "no error"


def test_there_is_no_cpu_fallback(core):
    """Without a GPU a launch fails loudly instead of computing on the host."""
    if core.is_active():
        pytest.skip("a CUDA device is present")
    assert not core.is_usable()
    assert "no CUDA device" in core.unusable_reason()
    with pytest.raises(RuntimeError, match="no CUDA device"):
        core.alloc_buffer(64)
    # a binary image needs the device too: an error, not a crash and not a host interpreter
    with pytest.raises(RuntimeError, match="no CUDA device"):
        core.load_metallib(b"\x7fELF" + bytes(128))
