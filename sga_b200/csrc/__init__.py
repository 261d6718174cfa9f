"""Loader for the native sm_100a library (``libsga_b200.so``).

``lib()`` returns the ``ctypes.CDLL`` handle, building the library first when
it is missing and ``nvcc`` is available. On a machine with a GPU the library is
mandatory: callers that reach a CUDA tensor without it get a loud
``RuntimeError`` instead of a silent PyTorch fallback.
"""
from __future__ import annotations

import ctypes
import os
import threading

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None
_LOCK = threading.Lock()


def lib_path() -> str:
    return os.path.join(_HERE, "libsga_b200.so")


def lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is not None:
        return _LIB
    with _LOCK:
        if _LIB is not None:
            return _LIB
        path = lib_path()
        if not os.path.exists(path):
            from . import build as _build

            path = _build.build()
        _LIB = ctypes.CDLL(path, mode=ctypes.RTLD_GLOBAL)
        _declare(_LIB)
        return _LIB


def available() -> bool:
    try:
        lib()
        return True
    except Exception:
        return False


_P = ctypes.c_void_p
_I = ctypes.c_int
_L = ctypes.c_longlong
_F = ctypes.c_float
_D = ctypes.c_double


def _declare(L: ctypes.CDLL) -> None:
    """Argument/return types of every exported launcher (all return int)."""
    sigs = {
        "sga_gemm_bf16": [_P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _I, _F, _P, _I, _P],
        "sga_gemm_bf16_pair": [_P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _I, _F, _P, _I, _P],
    }
    sigs.update(_EXTRA_SIGS)
    for name, args in sigs.items():
        try:
            fn = getattr(L, name)
        except AttributeError:
            continue
        fn.argtypes = args
        fn.restype = _I


# Filled in by the op wrapper modules' shared table below (kept in one place so
# a signature mismatch is a one-line fix).
_EXTRA_SIGS: dict = {}


def register_sigs(sigs: dict) -> None:
    _EXTRA_SIGS.update(sigs)
    if _LIB is not None:
        _declare(_LIB)
