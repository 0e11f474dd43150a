"""The Triton plugin's compile-and-launch path over the `tm_*` ABI, without Triton.

In the reference a kernel reaches the GPU through three pieces of its Triton plugin:
`MetalBackend.make_msl` (python/plugin/backend/compiler.py:131-146) turns the IR text into
`metal_args` - one `(index, kind, dtype)` per `tt.func` argument, read from `tm_kernel_info` -
and into the source `tm_emit_msl` returns; `MetalUtils.load_binary`
(python/plugin/backend/driver.py:31-40) makes the library and the pipeline; and
`MetalLauncher.__call__` (driver.py:58-92) builds the two arrays `tm_launch` takes from the
Python call's arguments and `metal_args`.  The plugin itself needs a Triton build this package
does not depend on, but none of the three pieces does: they only speak `_core`.  This module
restates them, so that a launch is marshalled from what `tm_kernel_info` reports - the only
thing the real plugin would consume - and not from a hand-written list of kinds.

`signature` is Triton's `src.signature`: parameter name -> type string in the order of the
Python definition, with "constexpr" for the parameters Triton specialised away (block sizes,
and integer arguments equal to 1, which is how the unit strides of a row-major matmul vanish
from the IR).
"""

import json

from . import _core

_INT_DTYPES = {"i1", "i8", "i16", "i32"}
_INT64_DTYPES = {"i64"}
_FLOAT_DTYPES = {"f32"}


def make_msl(ttir: str, num_warps: int = 4):
    """compiler.py:131-146 - (metadata, source bytes) for the first kernel of the module."""
    info = json.loads(_core.kernel_info(ttir, num_warps))
    kernel = info["kernels"][0]
    metadata = {
        "name": kernel["name"],
        "threads_per_threadgroup": kernel["threads_per_threadgroup"],
        "block_shape": kernel["block_shape"],
        "metal_args": [(a["index"], a["kind"], a["dtype"]) for a in kernel["args"]],
        "shared": 0,
    }
    return metadata, _core.emit_msl(ttir, num_warps).encode("utf-8")


def load_binary(name: str, image: bytes):
    """driver.py:31-40 - source bytes -> (library, pipeline, regs, spills, max threads)."""
    library = _core.compile_msl(image.decode("utf-8"))
    try:
        pipeline = _core.load_kernel(library, name)
    except Exception:
        _core.release_library(library)
        raise
    return library, pipeline, 0, 0, _core.kernel_max_threads(pipeline)


class Launcher:
    """driver.py:50-92 - marshals one launch; made once per compiled kernel."""

    def __init__(self, signature):
        # position in the Python call of each tt.func argument: the constexpr parameters are
        # in the call but not in the IR
        self.positions = [i for i, ty in enumerate(signature.values()) if ty != "constexpr"]

    def marshal(self, metal_args, args):
        kinds, values = [], []
        for index, kind, dtype in metal_args:
            arg = args[self.positions[index]]
            if kind == "pointer":
                handle = getattr(arg, "tm_handle", None)
                if handle is None:
                    raise TypeError(
                        f"argument {index} ({type(arg).__name__}) is not backed by device memory; "
                        "allocate it with triton_metal.buffer.MetalBuffer")
                kinds.append(_core.ARG_BUFFER)
                values.append(handle)
            elif dtype in _FLOAT_DTYPES:
                kinds.append(_core.ARG_F32)
                values.append(_core.float_bits(float(arg)))
            elif dtype in _INT_DTYPES:
                kinds.append(_core.ARG_I32)
                values.append(int(arg))
            elif dtype in _INT64_DTYPES:
                kinds.append(_core.ARG_I64)
                values.append(int(arg))
            else:
                raise TypeError(f"argument {index} has scalar type {dtype!r}; tm_launch carries "
                                "32-bit scalars and i64")
        return kinds, values

    def __call__(self, grid_0, grid_1, grid_2, function, packed_metadata, *args):
        _num_warps, threads, metal_args = packed_metadata
        kinds, values = self.marshal(metal_args, args)
        _core.launch(function, (grid_0, grid_1, grid_2), threads, kinds, values)


class CompiledKernel:
    """One kernel taken from IR text to a launchable, the way the plugin would:
    `CompiledKernel(ttir, signature)[grid](*python_call_arguments)`."""

    def __init__(self, ttir: str, signature, num_warps: int = 4):
        self.metadata, self.image = make_msl(ttir, num_warps)
        self.name = self.metadata["name"]
        self.library, self.function, _, _, self.max_threads = load_binary(self.name, self.image)
        self.launcher = Launcher(signature)
        self.packed_metadata = (num_warps, self.metadata["threads_per_threadgroup"],
                                self.metadata["metal_args"])

    def __getitem__(self, grid):
        grid = tuple(grid) + (1,) * (3 - len(grid))

        def run(*args):
            self.launcher(grid[0], grid[1], grid[2], self.function, self.packed_metadata, *args)

        return run

    def release(self):
        if self.function:
            _core.release_kernel(self.function)
            _core.release_library(self.library)
            self.function = self.library = 0
