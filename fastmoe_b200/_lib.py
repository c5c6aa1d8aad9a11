"""ctypes binding of `libfastmoe_b200.so` (the C ABI declared in include/fastmoe_b200.h).

The library is the only compute path of this package: there is no Python or
CPU fallback. Loading fails loudly when the shared object is missing and cannot
be built.
"""

from __future__ import annotations

import ctypes
import threading
from ctypes import c_char_p, c_int, c_int64, c_size_t, c_void_p

from . import build as _build

FMOE_F32, FMOE_BF16, FMOE_F16 = 0, 1, 2
FMOE_I64, FMOE_I32 = 0, 1

STATUS_BAD_INDEX = 1
STATUS_BAD_EXPERT = 2
STATUS_NULL_PTR = 4
STATUS_WAIT_TIMEOUT = 8

ACT_NONE, ACT_SWIGLU, ACT_GELU = 0, 1, 2

_P = c_void_p
_I = c_int
_L = c_int64

# name -> (restype, argtypes); mirrors include/fastmoe_b200.h one to one
SIGNATURES = {
    "fmoe_abi_version": (c_int, []),
    "fmoe_last_error": (c_char_p, []),
    "fmoe_status_name": (c_char_p, [_I]),
    "fmoe_tune": (c_int, [c_char_p, _I]),
    "fmoe_combine_scatter": (c_int, [_P, _P, _P, _P, _I, _P, _I, _P, _L, _L, _L, _L, _L, _I, _P, _P]),
    "fmoe_combine_plan_bytes": (c_size_t, [_L, _L]),
    "fmoe_combine_plan": (c_int, [_P, _P, _P, _P, _I, _P, _I, _L, _L, _L, _L, _I, _P, c_size_t, _P, _P]),
    "fmoe_combine_gather": (c_int, [_P, _P, _L, _L, _L, _L, _I, _I, _P]),
    "fmoe_combine_fwd_static": (c_int, [_P, _P, _P, _P, _I, _P, _I, _P, _L, _L, _L, _L, _L, _I, _I, _P, _P]),
    "fmoe_combine_bwd": (c_int, [_P, _P, _L, _P, _P, _L, _L, _L, _I, _P]),
    "fmoe_combine_routed": (c_int, [_P, _P, _P, _I, _P, _L, _L, _L, _L, _I, _I, _P]),
    "fmoe_combine_routed_bwd": (c_int, [_P, _P, _P, _I, _P, _L, _P, _P, _L, _L, _L, _I, _P]),
    "fmoe_route_topk": (c_int, [_P, _I, _L, _L, _L, _P, _P, _I, _P]),
    "fmoe_build_index_bytes": (c_size_t, [_L, _L, _L]),
    "fmoe_build_index": (c_int, [_P, _P, _I, _L, _L, _L, _L, _P, _P, _P, _P, _P, _P, _P, c_size_t, _P, _P]),
    "fmoe_permute_fwd": (c_int, [_P, _L, _P, _P, _L, _L, _L, _I, _P]),
    "fmoe_permute_bwd": (c_int, [_P, _P, _P, _L, _L, _L, _L, _I, _P]),
    "fmoe_grouped_gemm": (c_int, [_P, _P, _P, _P, _P, _P, _P, _L, _L, _L, _L, _I, _P, _P]),
    "fmoe_grouped_gemm_keep_pre": (c_int, [_P, _P, _P, _P, _P, _P, _P, _P, _L, _L, _L, _L, _I, _P, _P]),
    "fmoe_grouped_gemm_dgrad": (c_int, [_P, _P, _P, _P, _P, _P, _L, _L, _L, _L, _P, _P]),
    "fmoe_grouped_gemm_wgrad": (c_int, [_P, _P, _P, _P, _P, _L, _L, _L, _L, _P, _P]),
    "fmoe_swiglu_bwd": (c_int, [_P, _P, _P, _L, _L, _P]),
    "fmoe_gelu_bwd": (c_int, [_P, _P, _P, _L, _L, _P]),
    "fmoe_swiglu_bwd_ragged": (c_int, [_P, _P, _P, _L, _L, _P, _P]),
    "fmoe_permute_peer_fwd": (c_int, [_P, _L, _P, _P, _P, _P, _P, _L, _L, _L, _L, _L, _L, _P, _L, _L, _I, _P, _P]),
    "fmoe_peer_barrier": (c_int, [_P, _L, _L, ctypes.c_int32, _L, _P, _P]),
    "fmoe_ep_layout": (c_int, [_P, _L, _L, _L, _L, _L, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P]),
    "fmoe_combine_host_arena_bytes": (c_size_t, [_P, _L, _L, _L, _L, _I]),
    "fmoe_combine_host": (c_int, [_P, _P, _P, _I, _P, _I, _P, _L, _L, _L, _L, _I, _P, c_size_t, _P]),
}

_lock = threading.Lock()
_lib = None


class FastMoEError(RuntimeError):
    """A call into libfastmoe_b200.so returned a non-zero status."""

    def __init__(self, fn: str, status: int, message: str):
        self.fn, self.status = fn, status
        super().__init__(f"{fn} failed with status {status}: {message}")


def lib() -> ctypes.CDLL:
    """Loads (building first if needed) the shared library and binds every symbol."""
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                path = _build.ensure_built()
                handle = ctypes.CDLL(str(path))
                for name, (res, args) in SIGNATURES.items():
                    fn = getattr(handle, name)  # AttributeError if the export is missing
                    fn.restype = res
                    fn.argtypes = args
                _lib = handle
    return _lib


def call(name: str, *args):
    """Calls an int-returning entry point and raises on a non-zero status.

    Argument errors (status < 0) raise ValueError, CUDA errors (status > 0)
    raise FastMoEError.
    """
    handle = lib()
    status = getattr(handle, name)(*args)
    if status != 0:
        msg = handle.fmoe_last_error().decode("utf-8", "replace")
        if status < 0:
            raise ValueError(f"{name}: {msg} [{handle.fmoe_status_name(status).decode()}]")
        raise FastMoEError(name, status, msg)
    return status


def tune(key: str, value: int) -> None:
    call("fmoe_tune", key.encode(), int(value))
