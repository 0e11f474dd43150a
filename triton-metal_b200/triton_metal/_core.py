"""ctypes binding of libtmcuda's `tm_*` exports.

Mirrors python/triton_metal/_core.py:107-266 of the reference: one Python
function per export, the documented failure sentinel (NULL / 0 / -1) turned
into a RuntimeError that carries `tm_last_error`, and nothing computed here.
The library is found through TRITON_METAL_CORE_LIB (the reference's variable,
_core.py:40) or next to this package under ../lib.
"""

import ctypes
import os
import struct
from pathlib import Path

LIBRARY_NAME = "libtmcuda.so"


def library_path() -> str:
    """Where the shared library is expected; raises OSError when it is missing
    (there is no fallback implementation)."""
    candidates = [
        os.environ.get("TRITON_METAL_CORE_LIB"),
        str(Path(__file__).resolve().parents[1] / "lib" / LIBRARY_NAME),
    ]
    for candidate in candidates:
        if candidate and os.path.exists(candidate):
            return candidate
    raise OSError(
        f"{LIBRARY_NAME} not found (run `python __graft_entry__.py` or `make -C "
        "triton-metal_b200/csrc`, or set TRITON_METAL_CORE_LIB); looked in: "
        + ", ".join(c for c in candidates if c))


_lib = ctypes.CDLL(library_path())

_I32, _I64, _PTR, _STR = ctypes.c_int32, ctypes.c_int64, ctypes.c_void_p, ctypes.c_char_p
_I32P, _I64P = ctypes.POINTER(ctypes.c_int32), ctypes.POINTER(ctypes.c_int64)

#: (return type, argument types) of the 23 exports, as include/tm.h declares them.
EXPORTS = {
    "tm_version": (_PTR, ()),
    "tm_free": (None, (_PTR,)),
    "tm_last_error": (_PTR, ()),
    "tm_is_active": (_I32, ()),
    "tm_is_usable": (_I32, ()),
    "tm_unusable_reason": (_PTR, ()),
    "tm_device_name": (_PTR, ()),
    "tm_emit_msl": (_PTR, (_STR, _I32)),
    "tm_kernel_info": (_PTR, (_STR, _I32)),
    "tm_compile_msl": (_I64, (_STR,)),
    "tm_load_metallib": (_I64, (_PTR, _I64)),
    "tm_release_library": (_I32, (_I64,)),
    "tm_load_kernel": (_I64, (_I64, _STR)),
    "tm_kernel_max_threads": (_I64, (_I64,)),
    "tm_release_kernel": (_I32, (_I64,)),
    "tm_alloc_buffer": (_I64, (_I64,)),
    "tm_buffer_contents": (_PTR, (_I64,)),
    "tm_buffer_length": (_I64, (_I64,)),
    "tm_buffer_write": (_I32, (_I64, _I64, _PTR, _I64)),
    "tm_buffer_read": (_I32, (_I64, _I64, _PTR, _I64)),
    "tm_free_buffer": (_I32, (_I64,)),
    "tm_launch": (_I32, (_I64, _I64, _I64, _I64, _I64, _I32P, _I64P, _I32)),
    "tm_live_handle_count": (_I64, ()),
}

for _symbol, (_ret, _args) in EXPORTS.items():
    _entry = getattr(_lib, _symbol)      # a missing export fails the import
    _entry.restype = _ret
    _entry.argtypes = list(_args)


def _owned_text(address):
    """Decode and release a malloc'd string; None for NULL."""
    if not address:
        return None
    try:
        return ctypes.string_at(address).decode()
    finally:
        _lib.tm_free(address)


def last_error() -> str:
    return _owned_text(_lib.tm_last_error())


def _fail_if(result, sentinel):
    if result == sentinel:
        raise RuntimeError(last_error())
    return result


def _text_or_raise(address):
    text = _owned_text(address)
    if text is None:
        raise RuntimeError(last_error())
    return text


# -- device --------------------------------------------------------------------

def version() -> str:
    return _owned_text(_lib.tm_version())


def is_active() -> bool:
    return _lib.tm_is_active() != 0


def is_usable() -> bool:
    """True when a kernel of this library will actually run on this machine."""
    return _lib.tm_is_usable() != 0


def unusable_reason():
    return _owned_text(_lib.tm_unusable_reason())


def device_name():
    return _owned_text(_lib.tm_device_name())


# -- "compiler" ----------------------------------------------------------------

def emit_msl(ttir: str, num_simdgroups: int = 4) -> str:
    return _text_or_raise(_lib.tm_emit_msl(ttir.encode(), num_simdgroups))


def kernel_info(ttir: str, num_simdgroups: int = 4) -> str:
    return _text_or_raise(_lib.tm_kernel_info(ttir.encode(), num_simdgroups))


def compile_msl(source: str) -> int:
    return _fail_if(_lib.tm_compile_msl(source.encode()), 0)


def load_metallib(image: bytes) -> int:
    return _fail_if(_lib.tm_load_metallib(image, len(image)), 0)


def release_library(handle: int) -> None:
    _fail_if(_lib.tm_release_library(handle), -1)


# -- runtime -------------------------------------------------------------------

def load_kernel(library: int, name: str) -> int:
    return _fail_if(_lib.tm_load_kernel(library, name.encode()), 0)


def kernel_max_threads(kernel: int) -> int:
    return _fail_if(_lib.tm_kernel_max_threads(kernel), -1)


def release_kernel(handle: int) -> None:
    _fail_if(_lib.tm_release_kernel(handle), -1)


def alloc_buffer(nbytes: int) -> int:
    return _fail_if(_lib.tm_alloc_buffer(nbytes), 0)


def buffer_contents(handle: int) -> int:
    return _fail_if(_lib.tm_buffer_contents(handle), None)


def buffer_length(handle: int) -> int:
    return _fail_if(_lib.tm_buffer_length(handle), -1)


def buffer_write(handle: int, offset: int, address: int, nbytes: int) -> None:
    _fail_if(_lib.tm_buffer_write(handle, offset, ctypes.c_void_p(address), nbytes), -1)


def buffer_read(handle: int, offset: int, address: int, nbytes: int) -> None:
    _fail_if(_lib.tm_buffer_read(handle, offset, ctypes.c_void_p(address), nbytes), -1)


def free_buffer(handle: int) -> None:
    _fail_if(_lib.tm_free_buffer(handle), -1)


#: `tm_launch` argument kinds (Sources/TritonMetalCore/Compiler.swift:391-396).
ARG_BUFFER, ARG_I32, ARG_F32, ARG_I64 = 0, 1, 2, 3


def float_bits(value: float) -> int:
    """An f32 scalar travels as its bit pattern in the low 32 bits of a slot."""
    return struct.unpack("<I", struct.pack("<f", value))[0]


def pack_arguments(kinds, values):
    """The two parallel C arrays `tm_launch` takes."""
    count = len(kinds)
    if len(values) != count:
        raise ValueError("kinds and values differ in length")
    return (_I32 * count)(*kinds), (_I64 * count)(*values), count


def launch(kernel, grid, threads_per_threadgroup, kinds, values) -> None:
    """Run `kernel` over `grid` (three threadgroup counts) and wait for it."""
    kind_array, value_array, count = pack_arguments(kinds, values)
    _fail_if(
        _lib.tm_launch(kernel, grid[0], grid[1], grid[2], threads_per_threadgroup, kind_array,
                       value_array, count), -1)


def live_handle_count() -> int:
    return _lib.tm_live_handle_count()
