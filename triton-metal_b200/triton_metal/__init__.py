"""Host-side mirror of the reference's `triton_metal` shim over libtmcuda.

Same module and function names as python/triton_metal in the reference
(`_core` one function per `tm_*` export, `buffer.MetalBuffer`), so code written
against the reference's shim imports and runs unchanged; the additive `tmx_*`
entry points are reached through `triton_metal.cuda`.
"""

from . import _core  # noqa: F401
from .buffer import MetalBuffer  # noqa: F401

__all__ = ["_core", "MetalBuffer"]
