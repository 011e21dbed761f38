"""Tensor creation and weight initialisers. Parity: reference `genesis/init.py:14-373`.

CPU draws come from torch's global CPU generator (exactly what the reference's CPU
backend does, `genesis/ops/cpu/ops.py:291-339`, so seeded runs match it draw for
draw); CUDA draws come from the Philox kernels keyed by `genesis_b200.random`.
"""
import math

import numpy as np
import torch

from .device import as_torch_device
from .dtypes import get_dtype
from .tensor import Tensor
from .ops import dispatch as K
from . import random as _random


def _shape(shape):
    if len(shape) == 1 and isinstance(shape[0], (tuple, list, torch.Size)):
        return tuple(shape[0])
    return tuple(int(s) for s in shape)


def _mk(t, requires_grad):
    return Tensor._wrap(t, requires_grad=requires_grad)


def _draw(kind, shape, dtype, device, a, b):
    dev = as_torch_device(device)
    td = get_dtype(dtype).torch_dtype
    if dev.type == "cuda":
        seed, off = _random.default_generator().next_philox()
        return K.random_fill(kind, shape, td, dev, seed, off, a, b)
    if kind == "uniform":
        t = torch.rand(*shape, dtype=torch.float32)
        if (a, b) != (0.0, 1.0):
            t = t * (b - a) + a
    elif kind == "normal":
        t = torch.randn(*shape, dtype=torch.float32)
        if (a, b) != (0.0, 1.0):
            t = t * b + a
    else:
        return torch.randint(int(a), int(b), shape).to(td)
    return t.to(td)


def rand(*shape, low=0.0, high=1.0, device=None, dtype="float32", requires_grad=False):
    return _mk(_draw("uniform", _shape(shape), dtype, device, float(low), float(high)), requires_grad)


def randn(*shape, mean=0.0, std=1.0, device=None, dtype="float32", requires_grad=False):
    return _mk(_draw("normal", _shape(shape), dtype, device, float(mean), float(std)), requires_grad)


def randn_like(t, mean=0.0, std=1.0, requires_grad=False):
    return randn(*t.shape, mean=mean, std=std, device=t.device, dtype=t.dtype, requires_grad=requires_grad)


def randint(low, high=None, shape=None, *, size=None, device=None, dtype="int64", requires_grad=False):
    if high is None or isinstance(high, (tuple, list)):
        if isinstance(high, (tuple, list)):
            shape = high
        low, high = 0, low
    shape = size if size is not None else shape
    return _mk(_draw("randint", _shape((shape,)), dtype, device, low, high), False)


def randb(*shape, p=0.5, device=None, dtype="bool", requires_grad=False):
    """Bernoulli(p) mask: keeps where u <= p (reference `init.py:randb`)."""
    u = _draw("uniform", _shape(shape), "float32", device, 0.0, 1.0)
    return _mk((u <= p).to(get_dtype(dtype).torch_dtype), False)


def constant(*shape, c=1.0, device=None, dtype="float32", requires_grad=False):
    t = torch.empty(_shape(shape), dtype=get_dtype(dtype).torch_dtype, device=as_torch_device(device))
    K.fill_(t, c)
    return _mk(t, requires_grad)


def full(shape, fill_value, device=None, dtype="float32", requires_grad=False):
    if isinstance(shape, int):
        shape = (shape,)
    return constant(*shape, c=fill_value, device=device, dtype=dtype, requires_grad=requires_grad)


def ones(*shape, device=None, dtype="float32", requires_grad=False):
    return constant(*_shape(shape), c=1.0, device=device, dtype=dtype, requires_grad=requires_grad)


def zeros(*shape, device=None, dtype="float32", requires_grad=False):
    return constant(*_shape(shape), c=0.0, device=device, dtype=dtype, requires_grad=requires_grad)


def empty(*shape, device=None, dtype="float32", requires_grad=False):
    return _mk(torch.empty(_shape(shape), dtype=get_dtype(dtype).torch_dtype, device=as_torch_device(device)),
               requires_grad)


def _like(fn, t, dtype, device, requires_grad, **kw):
    return fn(*t.shape, device=device if device is not None else t.device,
              dtype=dtype if dtype is not None else t.dtype, requires_grad=requires_grad, **kw)


def empty_like(t, dtype=None, device=None, requires_grad=False):
    return _like(empty, t, dtype, device, requires_grad)


def zeros_like(t, dtype=None, device=None, requires_grad=False):
    return _like(zeros, t, dtype, device, requires_grad)


def ones_like(t, dtype=None, device=None, requires_grad=False):
    return _like(ones, t, dtype, device, requires_grad)


def full_like(t, fill_value, dtype=None, device=None, requires_grad=False):
    return _like(constant, t, dtype, device, requires_grad, c=fill_value)


def one_hot(n, i, device=None, dtype="float32", requires_grad=False):
    """`one_hot(num_classes, indices)` (reference argument order, `init.py:one_hot`)."""
    idx = i._t if isinstance(i, Tensor) else torch.as_tensor(i)
    out = torch.nn.functional.one_hot(idx.long(), int(n)).to(get_dtype(dtype).torch_dtype)
    if device is not None:
        out = out.to(as_torch_device(device))
    return _mk(out, requires_grad)


def eye(n, m=None, device=None, dtype="float32", requires_grad=False):
    return _mk(torch.eye(n, m if m is not None else n, dtype=get_dtype(dtype).torch_dtype,
                         device=as_torch_device(device)), requires_grad)


def arange(start, end=None, step=1, device=None, dtype=None, requires_grad=False):
    """Integer arguments give an exact int64 range; float arguments give float32."""
    if end is None:
        start, end = 0, start
    if dtype is None:
        is_int = all(isinstance(v, (int, np.integer)) for v in (start, end, step))
        dtype = "int64" if is_int else "float32"
    return _mk(K.arange(start, end, step, get_dtype(dtype).torch_dtype, as_torch_device(device)), requires_grad)


def from_numpy(array, device=None, dtype=None, requires_grad=False):
    arr = np.asarray(array)
    dt = get_dtype(dtype) if dtype is not None else get_dtype(arr.dtype)
    return Tensor(arr, dtype=dt, device=device if device is not None else "cpu", requires_grad=requires_grad)


def outer(a, b):
    from .nn import functional as F
    return F.matmul(F.reshape(a, (-1, 1)), F.reshape(b, (1, -1)))


def multinomial(probs, num_samples, replacement=False):
    p = probs._t.float()
    return _mk(torch.multinomial(p.cpu(), num_samples, replacement).to(p.device), False)


# ---- initialisers ------------------------------------------------------------------
def _fans(fan_in, fan_out, shape):
    if shape is not None:
        shape = tuple(shape)
        if len(shape) >= 2:
            rf = int(np.prod(shape[2:])) if len(shape) > 2 else 1
            return shape[1] * rf, shape[0] * rf, shape
        return shape[0], shape[0], shape
    return fan_in, fan_out, (fan_in, fan_out)


def xavier_uniform(fan_in, fan_out=None, gain=1.0, shape=None, **kw):
    fi, fo, shp = _fans(fan_in, fan_out, shape)
    a = gain * math.sqrt(6.0 / (fi + fo))
    return rand(*shp, low=-a, high=a, **kw)


def xavier_normal(fan_in, fan_out=None, gain=1.0, shape=None, **kw):
    fi, fo, shp = _fans(fan_in, fan_out, shape)
    return randn(*shp, mean=0.0, std=gain * math.sqrt(2.0 / (fi + fo)), **kw)


def kaiming_uniform(fan_in, fan_out=None, nonlinearity="relu", shape=None, **kw):
    fi, fo, shp = _fans(fan_in, fan_out, shape)
    bound = math.sqrt(2.0) * math.sqrt(3.0 / fi)
    return rand(*shp, low=-bound, high=bound, **kw)


def kaiming_normal(fan_in, fan_out=None, nonlinearity="relu", shape=None, **kw):
    fi, fo, shp = _fans(fan_in, fan_out, shape)
    return randn(*shp, mean=0.0, std=math.sqrt(2.0) / math.sqrt(fi), **kw)
