"""Device objects (`cpu`, `cuda`, `cuda:N`). Parity: reference `genesis/device.py:11-139`."""
from enum import Enum

import torch


class DeviceType(Enum):
    CPU = "cpu"
    CUDA = "cuda"


class Device:
    __slots__ = ("type", "index", "_torch")

    def __init__(self, spec="cpu", index=None):
        if isinstance(spec, Device):
            self.type, self.index = spec.type, spec.index
        elif isinstance(spec, torch.device):
            self.type = DeviceType(spec.type)
            self.index = spec.index if spec.index is not None else (0 if spec.type == "cuda" else None)
        elif isinstance(spec, DeviceType):
            self.type = spec
            self.index = (index or 0) if spec is DeviceType.CUDA else None
        elif isinstance(spec, int):
            self.type, self.index = DeviceType.CUDA, spec
        elif isinstance(spec, str):
            name, _, idx = spec.partition(":")
            if name not in ("cpu", "cuda"):
                raise ValueError(f"Unsupported device: {spec}")
            self.type = DeviceType(name)
            if name == "cuda":
                # a bare "cuda" is the process's current device (one process per GPU under torchrun)
                cur = torch.cuda.current_device() if torch.cuda.is_available() else 0
                self.index = int(idx) if idx else (index if index is not None else cur)
            else:
                self.index = None
        else:
            raise ValueError(f"Unsupported device spec: {spec!r}")
        self._torch = torch.device(self.type.value, self.index) if self.type is DeviceType.CUDA \
            else torch.device("cpu")

    @property
    def torch_device(self):
        return self._torch

    def is_cuda(self):
        return self.type is DeviceType.CUDA

    def is_cpu(self):
        return self.type is DeviceType.CPU

    def __eq__(self, other):
        if isinstance(other, str):
            try:
                other = Device(other)
            except ValueError:
                return False
        if isinstance(other, torch.device):
            other = Device(other)
        if not isinstance(other, Device):
            return False
        return self.type is other.type and (self.index or 0) == (other.index or 0)

    def __ne__(self, other):
        return not self.__eq__(other)

    def __hash__(self):
        return hash((self.type, self.index or 0))

    def __repr__(self):
        if self.type is DeviceType.CUDA:
            return f"cuda:{self.index}"
        return "cpu"

    __str__ = __repr__

    # Memory statistics documented for device objects (reference docs
    # `docs/en/api-reference/memory.md:9-118`); they forward to the cuda façade.
    def memory_allocated(self):
        from . import cuda
        return cuda.memory_allocated(self.index) if self.is_cuda() else 0

    def memory_reserved(self):
        from . import cuda
        return cuda.memory_reserved(self.index) if self.is_cuda() else 0

    memory_cached = memory_reserved

    def max_memory_allocated(self):
        from . import cuda
        return cuda.max_memory_allocated(self.index) if self.is_cuda() else 0

    def memory_stats(self):
        from . import cuda
        return cuda.memory_stats(self.index) if self.is_cuda() else {}

    def reset_memory_stats(self):
        from . import cuda
        if self.is_cuda():
            cuda.reset_max_memory_allocated(self.index)


_default_device = Device("cpu")


def device(spec="cpu", index=None):
    return spec if isinstance(spec, Device) else Device(spec, index)


def default_device():
    return _default_device


def set_default_device(dev):
    global _default_device
    _default_device = device(dev)


def cpu():
    return Device("cpu")


def cuda(index=0):
    return Device("cuda", index)


def as_torch_device(dev):
    """torch.device for None (default) / str / Device / torch.device."""
    if dev is None:
        return _default_device._torch
    if isinstance(dev, torch.device):
        return dev
    return device(dev)._torch
