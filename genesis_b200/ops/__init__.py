"""Kernel layer: `dispatch` (device routing on raw torch tensors) and `native` (ctypes
bindings of the sm_100a CUDA library built from `genesis_b200/csrc`)."""
from . import native, dispatch

__all__ = ["native", "dispatch"]
