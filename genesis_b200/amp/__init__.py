"""Automatic mixed precision. Parity: reference `genesis/amp/__init__.py:92-393`.

`autocast` switches the per-Function cast policy on (`function.py`); `GradScaler`
implements dynamic loss scaling.  Differences by design: the overflow flag stays on
the device (`found_inf`), the optimizer kernel unscales gradients on the fly and
skips itself on overflow, and `update()` adjusts the scale with device arithmetic,
so a training step has no host synchronisation (the reference reads `isfinite` back
every step, `amp/__init__.py:264-304`).  With `DistributedDataParallel` the unscale
and the overflow check are folded into the gradient all-reduce kernel.
"""
import torch

from ..amp_state import amp_state
from ..dtypes import get_dtype
from ..tensor import Tensor
from ..ops import dispatch as K
from ..function import AMPPolicy  # noqa: F401  (re-export)


class autocast:
    def __init__(self, device_type="cuda", enabled=True, dtype=None, cache_enabled=True):
        self.device_type = device_type
        self.enabled = enabled
        self.dtype = torch.float16 if dtype is None else get_dtype(dtype).torch_dtype
        self._prev = None

    def __enter__(self):
        self._prev = (amp_state.enabled, amp_state.dtype)
        amp_state.cache.clear()
        amp_state.enabled = bool(self.enabled)
        amp_state.dtype = self.dtype
        return self

    def __exit__(self, *exc):
        amp_state.enabled, amp_state.dtype = self._prev
        return False

    def __call__(self, fn):
        import functools

        @functools.wraps(fn)
        def wrapper(*a, **k):
            with autocast(self.device_type, self.enabled, self.dtype):
                return fn(*a, **k)
        return wrapper


def is_autocast_enabled():
    return amp_state.enabled


def get_autocast_dtype():
    return get_dtype(amp_state.dtype)


def clear_autocast_cache():
    amp_state.cache.clear()


class GradScaler:
    def __init__(self, init_scale=2.0 ** 16, growth_factor=2.0, backoff_factor=0.5, growth_interval=2000,
                 enabled=True, device=None):
        self._enabled = enabled
        self._init_scale = float(init_scale)
        self._growth_factor = growth_factor
        self._backoff_factor = backoff_factor
        self._growth_interval = growth_interval
        self._scale = None          # device fp32 [1]
        self._inv_scale = None
        self._growth_tracker = None  # device int32 [1]
        self._found_inf = None       # device fp32 [1]
        self._unscaled = set()
        self._stepped = False
        self._device = device
        # set by DistributedDataParallel when its fused all-reduce already unscaled the
        # gradients and raised the overflow flag for this step
        self._external_unscale = False

    # ---- lazy device state -----------------------------------------------------------
    def _lazy_init(self, device):
        if self._scale is None:
            self._scale = torch.full((1,), self._init_scale, dtype=torch.float32, device=device)
            self._growth_tracker = torch.zeros(1, dtype=torch.int32, device=device)
            self._found_inf = torch.zeros(1, dtype=torch.float32, device=device)

    def is_enabled(self):
        return self._enabled

    def get_scale(self):
        return self._init_scale if self._scale is None else float(self._scale.item())

    def scale(self, loss):
        if not self._enabled:
            return loss
        self._lazy_init(loss._t.device)
        from ..nn import functional as F
        return F.mul(loss, Tensor._wrap(self._scale.reshape(()).to(loss._t.dtype)))

    def _grads(self, optimizer):
        ps = [p for p in optimizer.params if p.grad is not None]
        # a data-parallel wrapper may have left the last bucket's all-reduce in flight (`overlap_optimizer`): anything
        # that reads the gradients waits for it first
        for j in {id(f): f for f in (getattr(p, "_late_join", None) for p in ps) if f is not None}.values():
            j()
        return [p.grad._t for p in ps]

    def unscale_(self, optimizer):
        """Divide the optimizer's gradients by the scale in place and record overflow."""
        if not self._enabled:
            return
        if id(optimizer) in self._unscaled:
            raise RuntimeError("unscale_() has already been called on this optimizer since the last update().")
        grads = self._grads(optimizer)
        if grads and not self._external_unscale:
            # (with DistributedDataParallel's fused all-reduce the gradients arrive here already divided by the scale
            # and checked for overflow: only the book-keeping below is left to do)
            self._lazy_init(grads[0].device)
            K.unscale_and_check(grads, 1.0 / self._scale, self._found_inf)
        self._unscaled.add(id(optimizer))

    def step(self, optimizer, *args, **kwargs):
        if not self._enabled:
            return optimizer.step(*args, **kwargs)
        grads = self._grads(optimizer)
        if not grads:
            return None
        self._lazy_init(grads[0].device)
        already = id(optimizer) in self._unscaled or self._external_unscale
        if not getattr(optimizer, "_fused_amp", False):
            # optimizer kernels without the scale / skip hooks: unscale in place, one host read of the flag
            if not already:
                K.unscale_and_check(grads, 1.0 / self._scale, self._found_inf)
                self._unscaled.add(id(optimizer))
            self._stepped = True
            return None if self.found_inf() else optimizer.step(*args, **kwargs)
        if already:
            optimizer._grad_scale = None          # already unscaled (explicitly or by the fused all-reduce)
        else:
            optimizer._grad_scale = 1.0 / self._scale
            # overflow check on the still-scaled gradients; the optimizer kernel multiplies by 1/scale
            K.unscale_and_check(grads, None, self._found_inf)
        optimizer._found_inf = self._found_inf
        try:
            ret = optimizer.step(*args, **kwargs)
        finally:
            optimizer._grad_scale = None
            optimizer._found_inf = None
        self._stepped = True
        return ret

    def update(self, new_scale=None):
        if not self._enabled or self._scale is None:
            return
        if new_scale is not None:
            self._scale.fill_(float(new_scale))
        else:
            f = self._found_inf
            # growth tracker and scale adjusted on the device: no readback
            grow = (self._growth_tracker + 1) * (f == 0).to(torch.int32)
            hit = (grow >= self._growth_interval)
            factor = torch.where(f > 0, torch.full_like(f, self._backoff_factor),
                                 torch.where(hit, torch.full_like(f, self._growth_factor), torch.ones_like(f)))
            self._scale.mul_(factor)
            self._growth_tracker.copy_(torch.where(hit, torch.zeros_like(grow), grow))
        self._found_inf.zero_()
        self._external_unscale = False
        self._unscaled.clear()
        self._stepped = False

    def found_inf(self):
        """Host read of the overflow flag (synchronises; for tests and logging)."""
        return self._found_inf is not None and float(self._found_inf.item()) != 0.0

    def state_dict(self):
        return {"scale": self.get_scale(), "growth_factor": self._growth_factor,
                "backoff_factor": self._backoff_factor, "growth_interval": self._growth_interval,
                "_growth_tracker": 0 if self._growth_tracker is None else int(self._growth_tracker.item())}

    def load_state_dict(self, state):
        self._init_scale = float(state["scale"])
        self._growth_factor = state["growth_factor"]
        self._backoff_factor = state["backoff_factor"]
        self._growth_interval = state["growth_interval"]
        if self._scale is not None:
            self._scale.fill_(self._init_scale)
            self._growth_tracker.fill_(int(state.get("_growth_tracker", 0)))


def get_amp_dtype(policy, *args, **kwargs):
    """Target dtype of an op under `policy` (None = no cast).  Parity: reference `amp/__init__.py:46-79`."""
    from .. import dtypes
    from ..function import AMPPolicy
    if policy == AMPPolicy.FP16:
        from ..amp_state import amp_state
        return dtypes.get_dtype(amp_state.dtype)
    if policy == AMPPolicy.FP32:
        return dtypes.float32
    if policy == AMPPolicy.PRESERVE:
        return None

    def has(value, names):
        if hasattr(value, "dtype") and getattr(value.dtype, "name", str(value.dtype)) in names:
            return True
        if isinstance(value, dict):
            return any(has(v, names) for v in value.values())
        if isinstance(value, (list, tuple)):
            return any(has(v, names) for v in value)
        return False

    low = ("float16", "bfloat16")
    if (has(args, ("float32",)) or has(kwargs, ("float32",))) and (has(args, low) or has(kwargs, low)):
        return dtypes.float32
    return None


def get_amp_cache():
    """The per-thread cache of low-precision parameter copies used inside `autocast`."""
    from ..amp_state import amp_state
    return amp_state.cache

from . import amp_cache  # noqa: E402,F401
