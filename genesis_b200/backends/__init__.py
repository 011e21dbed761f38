"""Storage layer names of the reference (`genesis.backends`: `Storage`, `CPUStorage`, `CUDAStorage`).

Tensors of this framework keep their bytes in a `torch.Tensor` (allocated by the native caching pool on CUDA), so
these classes are thin typed faces over one: they exist for code that builds tensors from storages or inspects a
tensor's storage (`shape / dtype / strides / ptr / nbytes`, `to_numpy`, `clone`, `contiguous`, indexing), with the
indexing and copies running through the same sm_100a kernels as the Tensor API.
Reference counterparts: `genesis/backends/base.py:13-60`, `backends/cpu.py:15-320`, `backends/cuda.py:188-1655`.
"""
from abc import ABC, abstractmethod

import numpy as np
import torch

from ..dtypes import DType, get_dtype

__all__ = ["Storage", "CPUStorage", "CUDAStorage"]


class Storage(ABC):
    """What every storage back end offers."""

    @abstractmethod
    def to_numpy(self):
        ...

    @abstractmethod
    def clone(self):
        ...

    @abstractmethod
    def contiguous(self):
        ...

    @abstractmethod
    def is_contiguous(self):
        ...

    @property
    @abstractmethod
    def shape(self):
        ...

    @property
    @abstractmethod
    def dtype(self):
        ...

    @abstractmethod
    def __getitem__(self, key):
        ...

    @abstractmethod
    def __setitem__(self, key, value):
        ...


class CPUStorage(torch.Tensor):
    """Host storage: a `torch.Tensor` subclass (as in the reference), plus the Storage interface."""

    def __new__(cls, data):
        if isinstance(data, torch.Tensor):
            return (data.cpu() if data.is_cuda else data).as_subclass(cls)
        if isinstance(data, np.ndarray):
            return torch.from_numpy(np.ascontiguousarray(data)).as_subclass(cls)
        return torch.tensor(data).as_subclass(cls)

    @classmethod
    def empty(cls, shape, dtype="float32"):
        return torch.empty(tuple(shape) if not isinstance(shape, int) else (shape,),
                           dtype=get_dtype(dtype).torch_dtype).as_subclass(cls)

    @classmethod
    def from_numpy(cls, arr, dtype=None):
        t = torch.from_numpy(np.ascontiguousarray(arr))
        if dtype is not None:
            t = t.to(get_dtype(dtype).torch_dtype)
        return t.as_subclass(cls)

    @classmethod
    def zeros(cls, shape, dtype=None):
        return torch.zeros(tuple(shape) if not isinstance(shape, int) else (shape,),
                           dtype=get_dtype(dtype or "float32").torch_dtype).as_subclass(cls)

    @classmethod
    def ones(cls, shape, dtype=None):
        return torch.ones(tuple(shape) if not isinstance(shape, int) else (shape,),
                          dtype=get_dtype(dtype or "float32").torch_dtype).as_subclass(cls)

    @property
    def strides(self):
        return tuple(self.stride())

    def to_cuda(self):
        return CUDAStorage.from_cpu_storage(self)

    def fill(self, value):
        self.fill_(value)
        return self

    def to_numpy(self):
        t = self.detach().as_subclass(torch.Tensor)
        return (t.float() if t.dtype == torch.bfloat16 else t).numpy()

    def numpy(self):
        return self.to_numpy()

    def clone(self):
        return torch.Tensor.clone(self).as_subclass(CPUStorage)

    def contiguous(self):
        return torch.Tensor.contiguous(self).as_subclass(CPUStorage)

    @property
    def size_bytes(self):
        return self.numel() * self.element_size()

    def data_ptr_int(self):
        return int(torch.Tensor.data_ptr(self))


Storage.register(CPUStorage)


class CUDAStorage(Storage):
    """Device storage: shape, dtype, strides and a device pointer over memory of the native pool."""

    def __init__(self, shape, dtype="float32", ptr=None, strides=None, base=None, stream=None, _tensor=None):
        if _tensor is not None:
            self._t = _tensor
        else:
            if isinstance(shape, int):
                shape = (shape,)
            flat = []
            for s in shape:
                flat.extend(s) if isinstance(s, (list, tuple)) else flat.append(s)
            shape = tuple(int(s) for s in flat)
            td = (dtype if isinstance(dtype, DType) else get_dtype(dtype)).torch_dtype
            if ptr is None:
                self._t = torch.empty(shape, dtype=td, device="cuda")
                if strides is not None and tuple(strides) != tuple(self._t.stride()):
                    self._t = torch.empty_strided(shape, tuple(strides), dtype=td, device="cuda")
            else:
                # a view over memory someone else owns (`base` keeps it alive)
                from ..distributed.symm import tensor_from_ptr
                n = 1
                for s in shape:
                    n *= s
                es = torch.empty(0, dtype=td).element_size()
                flat_t = tensor_from_ptr(int(ptr), max(n, 1) * es, td, torch.device("cuda", torch.cuda.current_device()))
                self._t = flat_t[:n].reshape(shape) if strides is None else flat_t.as_strided(shape, tuple(strides))
        self.base = base
        st = torch.cuda.current_stream().cuda_stream if stream is None else stream
        self.alloc_stream = self.last_stream = st
        self.recorded_streams = {st}
        self.owns_memory = ptr is None and base is None

    @classmethod
    def _wrap(cls, t, base=None):
        return cls(None, _tensor=t, base=base)

    @classmethod
    def from_cpu_storage(cls, cpu_storage, device_index=0):
        return cls._wrap(cpu_storage.as_subclass(torch.Tensor).to(f"cuda:{device_index}"))

    # ---- metadata --------------------------------------------------------------------
    @property
    def shape(self):
        return tuple(self._t.shape)

    @property
    def dtype(self):
        return get_dtype(self._t.dtype).name

    @property
    def dtype_obj(self):
        return get_dtype(self._t.dtype)

    @property
    def strides(self):
        return tuple(self._t.stride())

    @property
    def ptr(self):
        return self._t.data_ptr()

    def data_ptr(self):
        return self._t.data_ptr()

    @property
    def size(self):
        return self._t.numel()

    @property
    def itemsize(self):
        return self._t.element_size()

    def element_size(self):
        return self._t.element_size()

    @property
    def nbytes(self):
        return self._t.numel() * self._t.element_size()

    size_bytes = nbytes

    @property
    def ndim(self):
        return self._t.dim()

    def is_contiguous(self):
        return self._t.is_contiguous()

    def record_stream(self, stream):
        self.recorded_streams.add(stream)
        self.last_stream = stream

    # ---- data movement ------------------------------------------------------------------
    def to_numpy(self):
        t = self._t.detach()
        return (t.float() if t.dtype == torch.bfloat16 else t).cpu().numpy()

    numpy = to_numpy

    def from_numpy(self, arr):
        self._t.copy_(torch.from_numpy(np.ascontiguousarray(arr)).to(self._t.dtype).reshape(self._t.shape))
        return self

    def cpu(self):
        return CPUStorage(self._t.cpu())

    def copy_to_cuda(self, other):
        from ..ops import dispatch as K
        K.copy_(other._t, self._t.to(other._t.device))
        return other

    def clone(self):
        from ..ops import dispatch as K
        return CUDAStorage._wrap(K.clone(self._t))

    def contiguous(self):
        from ..ops import dispatch as K
        return self if self._t.is_contiguous() else CUDAStorage._wrap(K.contiguous(self._t))

    def fill(self, value):
        from ..ops import dispatch as K
        K.fill_(self._t, value)
        return self

    def to_dtype(self, dtype):
        from ..ops import dispatch as K
        return CUDAStorage._wrap(K.to_dtype(self._t, get_dtype(dtype).torch_dtype))

    # ---- views ------------------------------------------------------------------------------
    def reshape(self, *shape):
        shape = shape[0] if len(shape) == 1 and isinstance(shape[0], (tuple, list)) else shape
        return CUDAStorage._wrap(self._t.reshape(tuple(shape)), base=self)

    view = reshape

    def permute(self, *dims):
        dims = dims[0] if len(dims) == 1 and isinstance(dims[0], (tuple, list)) else dims
        return CUDAStorage._wrap(self._t.permute(tuple(dims)), base=self)

    def transpose(self, d0, d1):
        return CUDAStorage._wrap(self._t.transpose(d0, d1), base=self)

    def expand(self, *shape):
        shape = shape[0] if len(shape) == 1 and isinstance(shape[0], (tuple, list)) else shape
        return CUDAStorage._wrap(self._t.expand(tuple(shape)), base=self)

    # ---- indexing (same engine as Tensor.__getitem__ / __setitem__) ------------------------------
    def __getitem__(self, key):
        from ..ops import indexing
        key = _unwrap_key(key)
        return CUDAStorage._wrap(indexing.getitem(self._t, key), base=self)

    def __setitem__(self, key, value):
        from ..ops import indexing
        key = _unwrap_key(key)
        if isinstance(value, CUDAStorage):
            value = value._t
        elif isinstance(value, np.ndarray):
            value = torch.from_numpy(value).to(self._t.device, self._t.dtype)
        indexing.setitem_(self._t, key, value)

    # ---- the rest of the reference's storage surface -------------------------------------------------
    def numel(self):
        return self._t.numel()

    @property
    def device(self):
        from ..device import device as _device
        return _device(f"cuda:{self._t.device.index or 0}")

    @property
    def data(self):
        return self

    @property
    def T(self):
        return CUDAStorage._wrap(self._t.permute(*reversed(range(self._t.dim()))), base=self)

    def numpy_dtype(self):
        return np.float32 if self._t.dtype == torch.bfloat16 else torch.empty(0, dtype=self._t.dtype).numpy().dtype.type

    def stride(self, dim=None):
        return tuple(self._t.stride()) if dim is None else self._t.stride(dim)

    def share_memory_(self):
        """Device memory is visible to every thread of the process; cross-process sharing goes through the
        symmetric heap of `genesis.distributed.symm`."""
        return self

    def is_shared(self):
        return False

    def unsqueeze(self, dim):
        return CUDAStorage._wrap(self._t.unsqueeze(dim), base=self)

    def squeeze(self, dim=None):
        return CUDAStorage._wrap(self._t.squeeze() if dim is None else self._t.squeeze(dim), base=self)

    def broadcast_to(self, shape):
        return CUDAStorage._wrap(self._t.expand(tuple(shape)), base=self)

    def fill_(self, value):
        return self.fill(value)

    def item(self):
        if self._t.numel() != 1:
            raise ValueError("only one element tensors can be converted to Python scalars")
        return self._t.item()

    def to(self, target_dtype):
        return self.to_dtype(target_dtype)

    def float(self):
        return self.to_dtype("float32")

    def half(self):
        return self.to_dtype("float16")

    def long(self):
        return self.to_dtype("int64")

    def detach(self):
        return CUDAStorage._wrap(self._t.detach(), base=self)

    def copy_strided_to_contiguous(self, shape, stride, offset, dst_storage):
        """dst_storage (contiguous, `shape`) = the (shape, stride, offset) view of this storage's memory."""
        from ..ops import dispatch as K
        flat = self._t.reshape(-1) if self._t.is_contiguous() else self._t.contiguous().reshape(-1)
        K.copy_(dst_storage._t.reshape(tuple(shape)), flat.as_strided(tuple(shape), tuple(stride), int(offset)))
        return dst_storage

    def split(self, split_size_or_sections, dim=None):
        return [CUDAStorage._wrap(t, base=self) for t in torch.split(self._t, split_size_or_sections, dim or 0)]

    @staticmethod
    def cat(tensors, dim=0):
        from ..ops import dispatch as K
        return CUDAStorage._wrap(K.cat([t._t for t in tensors], dim))

    def __len__(self):
        return self._t.shape[0] if self._t.dim() else 0

    def __repr__(self):
        return f"CUDAStorage(shape={self.shape}, dtype={self.dtype}, ptr=0x{self.ptr:x})"


def _unwrap_key(key):
    if isinstance(key, CUDAStorage):
        return key._t
    if isinstance(key, tuple):
        return tuple(_unwrap_key(k) for k in key)
    return key

from . import base, base_storage, cpu, cuda, cuda_error, cuda_memory, cuda_utils  # noqa: E402,F401
