"""`genesis.backends.cuda` of the reference: `CUDAStorage` and the storage constructors `empty / zeros / ones /
from_numpy`.  (Its `IndexPlan` / `IndexKind` and strided-copy kernels are `ops/indexing.py` and `csrc/indexing.cu`,
`csrc/elementwise.cu` here.)"""
from enum import Enum

import numpy as np
import torch

from ..dtypes import get_dtype
from ..ops.indexing import Plan as IndexPlan  # noqa: F401
from . import CUDAStorage


class IndexKind(Enum):
    """Kinds of index plans of the reference's storage indexing; the planner here (`ops/indexing.py`) distinguishes
    views from kernel-backed gathers / scatters and reports them under these names."""
    VIEW = "view"
    GATHER = "gather"
    SCATTER = "scatter"
    COPY = "copy"
    FILL = "fill"
    MIXED_LIST_SLICE = "mixed_list_slice"


def _shape(shape):
    return tuple(shape[0]) if len(shape) == 1 and isinstance(shape[0], (list, tuple)) else tuple(shape)


def empty(*shape, dtype="float32", device_id=None):
    return CUDAStorage(_shape(shape), dtype)


def zeros(*shape, dtype="float32", device_id=None):
    s = CUDAStorage(_shape(shape), dtype)
    s.fill(0)
    return s


def ones(*shape, dtype="float32", device_id=None):
    s = CUDAStorage(_shape(shape), dtype)
    s.fill(1)
    return s


def from_numpy(arr, dtype=None):
    arr = np.ascontiguousarray(arr)
    t = torch.from_numpy(arr).to("cuda")
    if dtype is not None:
        t = t.to(get_dtype(dtype).torch_dtype)
    return CUDAStorage._wrap(t)
