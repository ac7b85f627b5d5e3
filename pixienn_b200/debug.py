"""Host side of the bounds-checked build of the library (include/pxe_debug.h).

``libpxe_checked.so`` (``python -m pixienn_b200._build --checked``) checks every global-memory access of every kernel
against a table of the caller's device allocations.  ``use_checked_library()`` makes this process load it instead of
``libpxe.so`` -- call it before anything else touches the library -- and re-arms the table from PyTorch's caching
allocator before every library call, so that every tensor alive at the call, with its exact requested size, is what
the kernels may touch.  ``read_report()`` returns what the kernels recorded.
"""
from __future__ import annotations

import ctypes as C
import os

import torch

from . import capi

CHECKED_LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "lib", "libpxe_checked.so")

_plain_lib = None


def live_allocations():
    """(address, bytes) of every block PyTorch's CUDA allocator has handed out and not taken back."""
    spans = []
    for seg in torch.cuda.memory_snapshot():
        for blk in seg["blocks"]:
            if blk["state"].startswith("active"):
                spans.append((int(blk["address"]), int(blk.get("requested_size", blk["size"]))))
    return spans


def set_allocations(spans) -> None:
    """Arms the check with these (address, bytes) ranges; an empty list disarms it."""
    L = _plain_lib() if _plain_lib else capi.lib()
    n = len(spans)
    starts = (C.c_void_p * max(n, 1))(*[a for a, _ in spans])
    sizes = (C.c_size_t * max(n, 1))(*[b for _, b in spans])
    capi.check(L.pxe_debug_set_allocations(starts, sizes, n))


def read_report(reset: bool = True) -> capi.BoundsReport:
    L = _plain_lib() if _plain_lib else capi.lib()
    rep = capi.BoundsReport()
    capi.check(L.pxe_debug_read_report(C.byref(rep), int(reset)))
    return rep


def describe(rep: capi.BoundsReport) -> str:
    kind = "store" if rep.is_store else "load"
    why = "misaligned" if rep.misaligned else "outside every allocation"
    return (f"{rep.violations} refused accesses; first: {rep.bytes}-byte {kind} at 0x{rep.address:x} ({why}), "
            f"{rep.file.decode(errors='replace')}:{rep.line}")


def use_checked_library() -> None:
    """Load the bounds-checked library in this process and arm it before every call made through ``capi.lib()``."""
    global _plain_lib
    if _plain_lib is not None:
        return
    if capi._lib is not None:
        raise RuntimeError("use_checked_library() must run before the library is first loaded")
    if not os.path.exists(CHECKED_LIB_PATH):
        raise ImportError(f"{CHECKED_LIB_PATH} is missing: build it with `python -m pixienn_b200._build --checked`")
    capi.LIB_PATH = CHECKED_LIB_PATH
    plain = capi.lib
    if plain().pxe_debug_bounds_checked() != 1:
        raise RuntimeError("libpxe_checked.so was not compiled with PXE_BOUNDS_CHECK")
    _plain_lib = plain

    class ArmedLibrary:
        """The loaded library; fetching an entry point first re-arms the table with the allocations alive now."""

        def __getattr__(self, name):
            L = plain()
            # (not while a stream is being captured into a CUDA graph: installing a table synchronises the device)
            if name.startswith("pxe_") and not name.startswith("pxe_debug_") and torch.cuda.is_available() \
                    and torch.cuda.is_initialized() and not torch.cuda.is_current_stream_capturing():
                set_allocations(live_allocations())
            return getattr(L, name)

    armed = ArmedLibrary()
    capi.lib = lambda: armed
