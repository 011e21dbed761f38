"""Loader of the native library (`genesis_b200/lib/libgenesis_b200.so`, built from `csrc/`
by `genesis_b200.build`).  On a machine with a GPU a missing library is an error, never a
silent fallback; on a CPU-only machine `get()` returns None and only CPU paths run."""
import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libgenesis_b200.so")

_lib = None
_tried = False


def get(required=None):
    """The ctypes handle, or None on CPU-only machines when the library is absent."""
    global _lib, _tried
    if _lib is not None:
        return _lib
    if required is None:
        required = torch.cuda.is_available()
    if not _tried or required:
        _tried = True
        if os.path.exists(LIB_PATH):
            _lib = ctypes.CDLL(LIB_PATH, mode=ctypes.RTLD_GLOBAL)
        elif required:
            raise RuntimeError(
                f"native library not found at {LIB_PATH}; build it with `python -m genesis_b200.build`")
    return _lib


def available():
    try:
        return get(required=False) is not None
    except OSError:
        return False
