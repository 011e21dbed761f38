"""`genesis.storage.Storage`: the unified storage container of the reference (`genesis/storage.py:12-220`): a back-end
storage (`CPUStorage` / `CUDAStorage`) plus its device, with allocation, numpy construction and device moves."""
import numpy as np
import torch

from .backends import CPUStorage, CUDAStorage
from .device import Device, device as make_device
from .dtypes import get_dtype


def _dev(d):
    if d is None:
        return make_device("cpu")
    return d if isinstance(d, Device) else make_device(d)


class Storage:
    def __init__(self, backend_storage, device):
        self._backend = backend_storage
        self.device = _dev(device)
        if isinstance(backend_storage, CUDAStorage):
            self.dtype = backend_storage.dtype
            self._size = backend_storage.size
            self.size_bytes = backend_storage.nbytes
        else:
            t = backend_storage
            self.dtype = str(t.dtype).replace("torch.", "")
            self._size = t.numel()
            self.size_bytes = t.numel() * t.element_size()

    @property
    def numel(self):
        return self._size

    @property
    def shape(self):
        return tuple(self._backend.shape)

    def element_size(self):
        return self._backend.element_size()

    def data_ptr(self):
        return int(self._backend.data_ptr())

    @classmethod
    def allocate(cls, size, dtype=None, device=None):
        dt = get_dtype(dtype)
        dev = _dev(device)
        shape = (size,) if isinstance(size, int) else tuple(size)
        backend = CPUStorage.empty(shape, dtype=dt.name) if dev.is_cpu() else CUDAStorage(shape, dt)
        return cls(backend, dev)

    @classmethod
    def make_storage(cls, numpy_data, dtype=None, device=None):
        if not isinstance(numpy_data, np.ndarray):
            raise ValueError(f"Storage.make_storage expects numpy array, got {type(numpy_data)}")
        dt = get_dtype(dtype)
        dev = _dev(device)
        if dev.is_cpu():
            return cls(CPUStorage.from_numpy(numpy_data, dtype=dt), dev)
        shape = numpy_data.shape if numpy_data.shape else (numpy_data.size,)
        return cls(CUDAStorage(shape, dt).from_numpy(numpy_data), dev)

    def __getitem__(self, index):
        if not self.device.is_cpu():
            raise RuntimeError("Cannot index GPU storage directly")
        return self._backend[index]

    def __setitem__(self, index, value):
        if not self.device.is_cpu():
            raise RuntimeError("Cannot assign to GPU storage directly")
        self._backend[index] = value

    def cpu(self):
        return self.to("cpu")

    def cuda(self, device=None):
        return self.to("cuda" if device is None else f"cuda:{device}")

    def to(self, target_device):
        target = _dev(target_device)
        if self.device == target:
            return self
        if self.device.is_cpu() and target.is_cuda():
            return Storage(CUDAStorage.from_cpu_storage(self._backend, target.index or 0), target)
        if self.device.is_cuda() and target.is_cpu():
            return Storage(self._backend.cpu(), target)
        moved = CUDAStorage._wrap(self._backend._t.to(f"cuda:{target.index or 0}"))
        return Storage(moved, target)

    def to_dtype(self, dtype):
        td = get_dtype(dtype).torch_dtype
        if isinstance(self._backend, CUDAStorage):
            return Storage(self._backend.to_dtype(dtype), self.device)
        return Storage(CPUStorage(self._backend.as_subclass(torch.Tensor).to(td)), self.device)

    def clone(self):
        return Storage(self._backend.clone(), self.device)

    def to_numpy(self):
        return self._backend.to_numpy()

    numpy = to_numpy

    def is_contiguous(self):
        return bool(self._backend.is_contiguous())
