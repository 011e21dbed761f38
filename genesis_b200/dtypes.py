"""Named dtype objects and conversions to/from numpy and torch.

API parity target: reference `genesis/dtypes.py:8-179` (DType objects comparable to
strings, `get_dtype` accepting DType / str / numpy / torch dtypes, `bfloat16`
travelling through numpy as float32).
"""
import builtins

import numpy as np
import torch


class DType:
    """A tensor element type. Compares equal to its own name as a string."""

    __slots__ = ("name", "itemsize", "numpy_dtype", "torch_dtype", "is_floating_point")

    def __init__(self, name, itemsize, numpy_dtype, torch_dtype, is_floating_point=None):
        self.name = name
        self.itemsize = itemsize
        self.numpy_dtype = numpy_dtype
        self.torch_dtype = torch_dtype
        if is_floating_point is None:
            is_floating_point = builtins.bool(np.issubdtype(numpy_dtype, np.floating))
        self.is_floating_point = is_floating_point

    def __repr__(self):
        return f"genesis.{self.name}"

    __str__ = __repr__

    def __eq__(self, other):
        if isinstance(other, DType):
            return self.name == other.name
        if isinstance(other, str):
            return self.name == other
        if isinstance(other, torch.dtype):
            return self.torch_dtype == other
        return False

    def __ne__(self, other):
        return not self.__eq__(other)

    def __hash__(self):
        return hash(self.name)

    def __reduce__(self):
        return (get_dtype, (self.name,))


float32 = DType("float32", 4, np.float32, torch.float32)
float16 = DType("float16", 2, np.float16, torch.float16)
float64 = DType("float64", 8, np.float64, torch.float64)
int32 = DType("int32", 4, np.int32, torch.int32)
int64 = DType("int64", 8, np.int64, torch.int64)
int16 = DType("int16", 2, np.int16, torch.int16)
int8 = DType("int8", 1, np.int8, torch.int8)
uint8 = DType("uint8", 1, np.uint8, torch.uint8)
bool = DType("bool", 1, np.bool_, torch.bool, is_floating_point=False)
# numpy has no bfloat16: host round trips go through float32 while itemsize stays 2.
bfloat16 = DType("bfloat16", 2, np.float32, torch.bfloat16, is_floating_point=True)

default_dtype = float32

_ALL = [float32, float16, float64, bfloat16, int32, int64, int16, int8, uint8, bool]
_name_to_dtype = {d.name: d for d in _ALL}
_name_to_dtype.update({"half": float16, "float": float32, "double": float64, "long": int64, "int": int32})
_torch_to_dtype = {d.torch_dtype: d for d in _ALL}
_numpy_to_dtype = {np.dtype(d.numpy_dtype): d for d in _ALL if d is not bfloat16}


def get_dtype(obj):
    """Normalise DType / name / numpy dtype / numpy scalar type / torch dtype to a DType.

    `None` maps to the default (float32).
    """
    if obj is None:
        return default_dtype
    if isinstance(obj, DType):
        return obj
    if isinstance(obj, str):
        try:
            return _name_to_dtype[obj]
        except KeyError:
            raise ValueError(f"Unknown dtype name: {obj}")
    if isinstance(obj, torch.dtype):
        try:
            return _torch_to_dtype[obj]
        except KeyError:
            raise ValueError(f"Unsupported torch dtype: {obj}")
    if obj is builtins.float:
        return float32
    if obj is builtins.int:
        return int64
    if obj is builtins.bool:
        return bool
    try:
        return _numpy_to_dtype[np.dtype(obj)]
    except (TypeError, KeyError):
        raise ValueError(f"Cannot interpret {obj!r} as a genesis dtype")


def to_torch_dtype(obj):
    return get_dtype(obj).torch_dtype


def is_floating_point(dtype):
    return get_dtype(dtype).is_floating_point


def is_integer(dtype):
    d = get_dtype(dtype)
    return (not d.is_floating_point) and d is not bool


def infer_dtype_from_data(data):
    """Dtype a Python/numpy payload would get (ints -> int64, floats -> float32)."""
    if isinstance(data, builtins.bool):
        return bool
    if isinstance(data, builtins.int):
        return int64
    if isinstance(data, builtins.float):
        return float32
    if isinstance(data, np.ndarray) or isinstance(data, np.generic):
        if data.dtype == np.float64:
            return float32
        return get_dtype(data.dtype)
    if isinstance(data, torch.Tensor):
        return get_dtype(data.dtype)
    if isinstance(data, (list, tuple)):
        arr = np.asarray(data)
        if arr.dtype == np.float64:
            return float32
        if arr.dtype == np.bool_:
            return bool
        if np.issubdtype(arr.dtype, np.integer):
            return int64
        return get_dtype(arr.dtype)
    return default_dtype


# Lists kept for API parity with the reference (`dtypes.py:183-185`).
all_dtypes = [float32, float16, float64, bfloat16, int32, int64, int16, int8, uint8, bool]
floating_dtypes = [dt for dt in all_dtypes if dt.is_floating_point]
integer_dtypes = [dt for dt in all_dtypes if not dt.is_floating_point and dt is not bool]
