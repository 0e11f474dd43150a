"""Bindings of libtmcuda's additive `tmx_*` entry points (no counterpart in the
reference): device selection, kernel options, asynchronous and timed launches."""

import ctypes

from . import _core

_lib = _core._lib
_I32, _I64, _PTR, _STR = ctypes.c_int32, ctypes.c_int64, ctypes.c_void_p, ctypes.c_char_p
_I32P, _I64P, _F32P = (ctypes.POINTER(ctypes.c_int32), ctypes.POINTER(ctypes.c_int64),
                       ctypes.POINTER(ctypes.c_float))

_LAUNCH = (_I64, _I64, _I64, _I64, _I64, _I32P, _I64P, _I32)

EXPORTS = {
    "tmx_set_device": (_I32, (_I32,)),
    "tmx_get_device": (_I32, ()),
    "tmx_sm_count": (_I32, ()),
    "tmx_kernel_set_option": (_I32, (_I64, _STR, _I64)),
    "tmx_kernel_last_path": (_I32, (_I64,)),
    "tmx_launch_async": (_I32, _LAUNCH),
    "tmx_launch_timed": (_I32, _LAUNCH + (_I32, _F32P)),
    "tmx_synchronize": (_I32, ()),
    "tmx_buffer_write_async": (_I32, (_I64, _I64, _PTR, _I64)),
    "tmx_buffer_read_async": (_I32, (_I64, _I64, _PTR, _I64)),
    "tmx_buffer_fill": (_I32, (_I64, _I64, _I32, _I64)),
    "tmx_timer_begin": (_I32, ()),
    "tmx_timer_end": (_I32, (_F32P,)),
    "tmx_launch_count": (_I64, ()),
    "tmx_alloc_device_buffer": (_I64, (_I64,)),
    "tmx_buffer_device_pointer": (_PTR, (_I64,)),
    "tmx_stream_handle": (_PTR, ()),
    "tmx_matmul_f32_static": (_I32, (_I64,) * 12),
    "tmx_matmul_f32_static_capacity": (_I64, ()),
    "tmx_matmul_f32_static_prepare": (_I32, ()),
    "tmx_device_memory": (_I32, (_I64P, _I64P)),
    "tmx_ipc_export": (_I32, (_I64, _PTR)),
    "tmx_ipc_import": (_I64, (_PTR, _I64)),
    "tmx_gather_flag_bytes": (_I64, ()),
    "tmx_matmul_gathered": (_I32, (_I64, _I64, _I64, _I64P, _I64P, _I32, _I32, _I64, _I64, _I64, _I64, _I32,
                                   ctypes.c_uint32, _I32)),
    "tmx_debug_attention_schedule": (_I64, (_I32, _I32, _I32, _I32, _I32, _I32, _I32P, _I64, _I32P, _I64P)),
    "tmx_selftest_bounded_wait": (_I32, (_I64, _I32P)),
    "tmx_debug_inject_status": (_I32, (_I32, _I32, _I32, _I32)),
}

for _symbol, (_ret, _args) in EXPORTS.items():
    _entry = getattr(_lib, _symbol)
    _entry.restype = _ret
    _entry.argtypes = list(_args)

PATH_AUTO, PATH_SIMT, PATH_TCGEN05 = 0, 1, 2


def _ok(status):
    if status == -1:
        raise RuntimeError(_core.last_error())
    return status


def set_device(ordinal: int) -> None:
    _ok(_lib.tmx_set_device(ordinal))


def get_device() -> int:
    return _ok(_lib.tmx_get_device())


def sm_count() -> int:
    return _ok(_lib.tmx_sm_count())


def set_option(kernel: int, name: str, value: int) -> None:
    _ok(_lib.tmx_kernel_set_option(kernel, name.encode(), value))


def last_path(kernel: int) -> int:
    return _ok(_lib.tmx_kernel_last_path(kernel))


def launch_async(kernel, grid, threads, kinds, values) -> None:
    k, v, n = _core.pack_arguments(kinds, values)
    _ok(_lib.tmx_launch_async(kernel, grid[0], grid[1], grid[2], threads, k, v, n))


def launch_timed(kernel, grid, threads, kinds, values, repeats: int) -> float:
    """Milliseconds for `repeats` back-to-back launches (CUDA events on the
    library's stream)."""
    k, v, n = _core.pack_arguments(kinds, values)
    elapsed = ctypes.c_float(0.0)
    _ok(_lib.tmx_launch_timed(kernel, grid[0], grid[1], grid[2], threads, k, v, n, repeats,
                              ctypes.byref(elapsed)))
    return elapsed.value


def synchronize() -> None:
    _ok(_lib.tmx_synchronize())


def write_async(handle, offset, address, nbytes) -> None:
    _ok(_lib.tmx_buffer_write_async(handle, offset, ctypes.c_void_p(address), nbytes))


def read_async(handle, offset, address, nbytes) -> None:
    _ok(_lib.tmx_buffer_read_async(handle, offset, ctypes.c_void_p(address), nbytes))


def fill(handle, offset, byte, nbytes) -> None:
    _ok(_lib.tmx_buffer_fill(handle, offset, byte, nbytes))


def timer_begin() -> None:
    _ok(_lib.tmx_timer_begin())


def timer_end() -> float:
    elapsed = ctypes.c_float(0.0)
    _ok(_lib.tmx_timer_end(ctypes.byref(elapsed)))
    return elapsed.value


def launch_count() -> int:
    return _lib.tmx_launch_count()


def matmul_f32_static(a, b, c, M, N, K, strides=None) -> None:
    """fp32 C = A @ B through the entry point that allocates nothing (scratch in a
    fixed device array; see include/tm.h for the size limit)."""
    if strides is None:
        strides = (K, 1, N, 1, N, 1)
    _ok(_lib.tmx_matmul_f32_static(a, b, c, M, N, K, *strides))


def matmul_f32_static_capacity() -> int:
    return _lib.tmx_matmul_f32_static_capacity()


def alloc_device_buffer(nbytes: int) -> int:
    """A buffer of plain device memory (no host pointer); free it with _core.free_buffer."""
    handle = _lib.tmx_alloc_device_buffer(nbytes)
    if handle == 0:
        raise RuntimeError(_core.last_error())
    return handle


def device_pointer(handle: int) -> int:
    address = _lib.tmx_buffer_device_pointer(handle)
    if not address:
        raise RuntimeError(_core.last_error())
    return address


def stream_handle() -> int:
    """The library's cudaStream_t as an integer (for torch.cuda.ExternalStream)."""
    return _lib.tmx_stream_handle() or 0


def selftest_bounded_wait(budget_cycles: int):
    """Run the kernel whose waits are meant to run out; returns what its two waits reported
    (1 = gave up).  The device status word stays set for the next synchronising call."""
    results = (ctypes.c_int32 * 2)()
    _ok(_lib.tmx_selftest_bounded_wait(budget_cycles, results))
    return results[0], results[1]


def inject_status(code: int, where: int = 0, block: int = 0, extra: int = 0) -> None:
    _ok(_lib.tmx_debug_inject_status(code, where, block, extra))


def matmul_f32_static_prepare() -> None:
    _ok(_lib.tmx_matmul_f32_static_prepare())


def device_memory():
    """(free, total) bytes of device memory."""
    free, total = ctypes.c_int64(0), ctypes.c_int64(0)
    _ok(_lib.tmx_device_memory(ctypes.byref(free), ctypes.byref(total)))
    return free.value, total.value


def ipc_export(handle: int) -> bytes:
    """The 64-byte token with which another process maps this device buffer."""
    token = ctypes.create_string_buffer(64)
    _ok(_lib.tmx_ipc_export(handle, token))
    return token.raw


def ipc_import(token: bytes, nbytes: int) -> int:
    handle = _lib.tmx_ipc_import(bytes(token), nbytes)
    if handle == 0:
        raise RuntimeError(_core.last_error())
    return handle


def gather_flag_bytes() -> int:
    return _lib.tmx_gather_flag_bytes()


def matmul_gathered(kernel, a, b, replicas, flags, rank, row0, rows, N, K, slot, epoch, wait=True) -> None:
    world = len(replicas)
    c_arr = (ctypes.c_int64 * world)(*replicas)
    f_arr = (ctypes.c_int64 * world)(*flags)
    _ok(_lib.tmx_matmul_gathered(kernel, a, b, c_arr, f_arr, world, rank, row0, rows, N, K, slot, epoch,
                                 1 if wait else 0))


def attention_schedule(kind: str, bh: int, rows: int, n_ctx: int, causal: bool, ctas: int):
    """The per-CTA work lists of a persistent attention kernel: (lists, loads) where lists[c] is
    CTA c's sequence of (batch-head, block) pairs and loads[c] its modelled cost."""
    code = {"fwd": 0, "dq": 1, "dkdv": 2}[kind]
    block_rows = 256 if code == 0 else 128
    capacity = bh * ((rows + block_rows - 1) // block_rows)
    items = (ctypes.c_int32 * (2 * capacity))()
    begin = (ctypes.c_int32 * (ctas + 1))()
    load = (ctypes.c_int64 * ctas)()
    n = _lib.tmx_debug_attention_schedule(code, bh, rows, n_ctx, int(causal), ctas, items, capacity, begin, load)
    if n < 0:
        raise RuntimeError(_core.last_error())
    used = min(ctas, n)
    lists = [[(items[2 * i], items[2 * i + 1]) for i in range(begin[c], begin[c + 1])] for c in range(used)]
    return lists, list(load)[:used]
