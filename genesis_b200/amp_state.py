"""Thread-local autocast state shared by `function.py` and `amp/`.

The reference keeps these flags as process-global module attributes
(`genesis/__init__.py:16-18`); here they are thread-local so a data-loader or
watchdog thread can never observe another thread's autocast region.
"""
import threading
import weakref

import torch


class _AmpState(threading.local):
    def __init__(self):
        self.enabled = False
        self.dtype = torch.float16
        self.cache = {}


class ShadowEntry:
    """A persistent low-precision copy of a parameter, kept current by the optimizer kernel (see
    `optim.Optimizer.enable_shadows`).  `version` is the parameter's `_version` at the last refresh: any in-place
    change through the Tensor API makes the entry stale and the autocast cast falls back to a conversion."""
    __slots__ = ("param", "lp", "version", "group", "__weakref__")

    def __init__(self, param, lp, group):
        self.param, self.lp, self.version, self.group = param, lp, param._version, group

    def valid(self, raw, dtype):
        p = self.param
        return p._t is raw and self.version == p._version and self.lp.dtype == dtype


# fp32 parameter storage address -> ShadowEntry (process-wide: parameters are shared between threads).  The optimizer
# that maintains the copies owns the entries; they leave this table when it is collected.
shadows = weakref.WeakValueDictionary()


def shadow_of(raw, dtype):
    """The current low-precision copy of the parameter whose storage is `raw`, or None."""
    if not shadows:
        return None
    e = shadows.get(raw.data_ptr())
    return e.lp if e is not None and e.valid(raw, dtype) else None


def stacked_shadow_of(raws, dtype):
    """When `raws` are exactly the members of one shadow group, in order, and all current: the group's stacked
    low-precision buffer (rows of the members one after another).  None otherwise."""
    if not shadows:
        return None
    first = shadows.get(raws[0].data_ptr())
    if first is None or first.group is None:
        return None
    members, buf = first.group
    if len(members) != len(raws):
        return None
    for e, r in zip(members, raws):
        if not e.valid(r, dtype):
            return None
    return buf


# address of a low-precision weight copy [N, K] (or of a group's stacked buffer) -> its transposed twin [K, N], kept
# current by the same optimizer step that refreshes the copy.  The data-gradient GEMM of a linear layer reads the twin
# so that both of its operands are contiguous along the contraction (the layout the tensor cores read fastest).
transposed = {}


def transposed_of(lp):
    """The [K, N] twin of the low-precision weight `lp` [N, K] when the optimizer maintains one, else None."""
    if not transposed:
        return None
    t = transposed.get(lp.data_ptr())
    if t is None or t.dtype != lp.dtype or t.dim() != 2 or lp.dim() != 2 or t.shape[0] != lp.shape[1] \
            or t.shape[1] != lp.shape[0]:
        return None
    return t


amp_state = _AmpState()
