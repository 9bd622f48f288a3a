"""Loads ``libkb200.so`` (the sm_100a kernels) through ``ctypes``.

On a machine with a CUDA device the library must be present or buildable; a missing library raises
(a silent fallback to library kernels would hide a broken build).  On CPU-only machines ``get()``
returns ``None`` and every op uses its torch path.
"""

import ctypes
import os
import threading

import torch

_LIB = None
_LOCK = threading.Lock()
_TRIED = False


def available():
    return torch.cuda.is_available()


def get():
    """The loaded library, or ``None`` when there is no CUDA device."""
    global _LIB, _TRIED
    if _LIB is not None:
        return _LIB
    if not torch.cuda.is_available():
        return None
    with _LOCK:
        if _LIB is None:
            from keras_b200.kernels import build

            path = build.LIB_PATH
            if not build.is_current():
                path = build.build()
            _LIB = ctypes.CDLL(path)
            _declare(_LIB)
    return _LIB


def get_for_symbols():
    """Load the library without requiring a device (symbol inspection, build checks)."""
    from keras_b200.kernels import build

    path = build.build()
    lib = ctypes.CDLL(path)
    return lib


def _declare(lib):
    vp, i32, i64, f32 = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
    sigs = {
        "kb200_last_error": ([], ctypes.c_char_p),
    }
    for name, (args, res) in sigs.items():
        if hasattr(lib, name):
            fn = getattr(lib, name)
            fn.argtypes = args
            fn.restype = res


def stream_ptr():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def check(code, what):
    if code != 0:
        lib = get()
        msg = lib.kb200_last_error().decode() if lib is not None and hasattr(lib, "kb200_last_error") else ""
        raise RuntimeError(f"kernel launch failed in {what}: code {code} {msg}")
