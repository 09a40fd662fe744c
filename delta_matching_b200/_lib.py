"""ctypes binding of the C ABI in include/dm_b200.h.

The library is `libdm_b200.so` next to this file (built by `python -m delta_matching_b200.build`) or the file named by
the environment variable DM_SO.  Nothing else is ever loaded in its place and there is no fallback: a missing library
raises RuntimeError.  Mirrors the loader contract of delta_matching/core.py:81-104 (DM_SO override, refuse a missing
library, load once).
"""
from __future__ import annotations

import ctypes
import os
import threading

_LOCK = threading.Lock()
_LIB = None
_PATH = None

_P = ctypes.c_void_p
_I = ctypes.c_int
_L = ctypes.c_int64
_F = ctypes.c_float

# name -> (restype, argtypes); the single source of truth the symbol test checks against include/dm_b200.h
SIGNATURES = {
    "dm_version": (_I, []),
    "dm_numerics": (ctypes.c_char_p, []),
    "dm_last_error": (_I, [ctypes.c_char_p, _I]),
    "dm_quant_qkv_workspace_bytes": (ctypes.c_size_t, [_I, _I, _I, _I]),
    "dm_kmean": (_I, [_P, _L, _L, _L, _I, _I, _I, _I, _P, _P, _P]),
    "dm_quant_rows": (_I, [_P, _L, _L, _L, _P, _F, _P, _L, _L, _L, _I, _I, _I, _I, _P, _P, _P, _P]),
    "dm_quant_qkv": (_I, [_P, _L, _L, _L, _P, _L, _L, _L, _P, _L, _L, _L, _I, _I, _I, _I, _I,
                          _P, _P, _P, _P, _P, _P, _P, _P, _P]),
    "dm_quant_do": (_I, [_P, _L, _L, _L, _P, _L, _L, _L, _I, _I, _I, _I, _P, _P, _P, _P]),
    "dm_fwd": (_I, [_P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P, _L, _L, _L, _P, _P, _P]),
    "dm_dbg_fwd_unordered": (_I, [_P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P, _L, _L, _L, _P, _P, _P]),
    "dm_delta": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P, _P, _P]),
    "dm_delta_sum": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P, _P, _P]),
    "dm_bwd": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I,
                    _P, _L, _L, _L, _P, _L, _L, _L, _P, _L, _L, _L, _P, _P, _P, _P]),
    "dm_bwd_parts": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I,
                          _P, _L, _L, _L, _P, _L, _L, _L, _P, _L, _L, _L, _P, _P, _I, _P, _P]),
    "dm_bwd_workspace_bytes": (_L, [_I, _I, _I, _I]),
    "dm_bwd_ws": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I,
                       _P, _L, _L, _L, _P, _L, _L, _L, _P, _L, _L, _L, _P, _L, _I, _P, _P]),
    "dm_dbg_mma_tile": (_I, [_P, _P, _P, _P, _I, _I, _I, _I, _I, _P, _P, _P]),
    "dm_dbg_wait_expiry": (_I, [_P, _P, _P, ctypes.c_longlong, _P, _P]),
    "dm_launch_count": (ctypes.c_longlong, []),
    "dm_copy_2d_async": (_I, [_P, _L, _P, _L, _L, _L, _I, _P]),
    "dm_kmean_static": (_I, [_P, _L, _L, _L, _I, _I, _I, _I, _P, _P, ctypes.c_char_p, _I]),
}


def library_path() -> str:
    so = os.environ.get("DM_SO")
    if so:
        if not os.path.isfile(so):
            raise RuntimeError(f"DM_SO={so!r} does not exist")
        return so
    here = os.path.dirname(os.path.abspath(__file__))
    so = os.path.join(here, "libdm_b200.so")
    if not os.path.isfile(so):
        raise RuntimeError("delta_matching_b200: libdm_b200.so is not built: run `python -m delta_matching_b200.build` "
                           "in the checkout, or point DM_SO at a built library (there is no fallback path)")
    return so


def lib():
    """The loaded library (loaded once; raises RuntimeError if it is missing or lacks a symbol)."""
    global _LIB, _PATH
    if _LIB is None:
        with _LOCK:
            if _LIB is None:
                path = library_path()
                handle = ctypes.CDLL(path)
                for name, (res, args) in SIGNATURES.items():
                    try:
                        fn = getattr(handle, name)
                    except AttributeError as e:
                        raise RuntimeError(f"delta_matching_b200: {path} does not export {name}") from e
                    fn.restype = res
                    fn.argtypes = args
                _PATH = path
                _LIB = handle
    return _LIB


def loaded_library():
    """Path of the loaded shared library (None before the first lib() call)."""
    return _PATH


def last_error() -> str:
    buf = ctypes.create_string_buffer(1024)
    lib().dm_last_error(buf, 1024)
    return buf.value.decode("utf-8", "replace")


def check(rc: int) -> None:
    """Raise RuntimeError with the library's message for a non-zero return code (the op-level error type of the
    reference, csrc/delta_matching_api.cpp:73-98 via TORCH_CHECK)."""
    if rc != 0:
        raise RuntimeError(last_error() or f"delta_matching_b200: library call failed with code {rc}")
