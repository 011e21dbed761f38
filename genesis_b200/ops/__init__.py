"""Kernel layer: `dispatch` (device routing on raw torch tensors) and `native` (ctypes
bindings of the sm_100a CUDA library built from `genesis_b200/csrc`)."""
from . import native, dispatch
from .dispatcher import OperationDispatcher  # noqa: F401  (the reference exports it, with DeviceType, from `genesis.ops`)
from ..device import DeviceType  # noqa: F401

__all__ = ["native", "dispatch", "OperationDispatcher", "DeviceType"]
