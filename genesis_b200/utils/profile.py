"""Wall-clock profiling decorator and CUDA-event timers.

`profile` mirrors reference `genesis/utils/profile.py:14-72` (per-function / per-class totals
printed at exit).  `CudaTimer` and `nvtx_range` add device-side timing: CUDA events on the
launching stream, and NVTX ranges around Functions when `GENESIS_NVTX=1`.
"""
import atexit
import contextlib
import functools
import os
import time
from collections import defaultdict

import torch

_totals = defaultdict(lambda: [0, 0.0])
_enabled_print = False


def _report():
    if _totals and _enabled_print:
        print("\n=== genesis_b200 profile ===")
        for name, (n, t) in sorted(_totals.items(), key=lambda kv: -kv[1][1]):
            print(f"{name}: {n} calls, {t:.6f}s total, {t / max(n, 1) * 1e3:.3f} ms/call")


atexit.register(_report)


def _wrap_fn(fn, name):
    @functools.wraps(fn)
    def wrapper(*a, **k):
        t0 = time.perf_counter()
        try:
            return fn(*a, **k)
        finally:
            rec = _totals[name]
            rec[0] += 1
            rec[1] += time.perf_counter() - t0
    return wrapper


def profile(obj):
    """Decorator for a function or a class (wraps every public method)."""
    global _enabled_print
    _enabled_print = True
    if isinstance(obj, type):
        for k, v in list(vars(obj).items()):
            if callable(v) and not k.startswith("__"):
                setattr(obj, k, _wrap_fn(v, f"{obj.__name__}.{k}"))
        return obj
    return _wrap_fn(obj, getattr(obj, "__qualname__", str(obj)))


def get_profile_data():
    return {k: tuple(v) for k, v in _totals.items()}


def reset_profile():
    _totals.clear()


class CudaTimer:
    """Named regions timed with CUDA events on the current stream; `summary()` synchronises once."""

    def __init__(self):
        self._pairs = defaultdict(list)

    @contextlib.contextmanager
    def region(self, name):
        if not torch.cuda.is_available():
            t0 = time.perf_counter()
            yield
            self._pairs[name].append((time.perf_counter() - t0) * 1e3)
            return
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        yield
        b.record()
        self._pairs[name].append((a, b))

    def summary(self):
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        out = {}
        for name, items in self._pairs.items():
            ms = [x if isinstance(x, float) else x[0].elapsed_time(x[1]) for x in items]
            out[name] = {"calls": len(ms), "total_ms": sum(ms), "mean_ms": sum(ms) / max(len(ms), 1)}
        return out


_NVTX = os.environ.get("GENESIS_NVTX", "0") == "1"


@contextlib.contextmanager
def nvtx_range(name):
    if _NVTX and torch.cuda.is_available():
        torch.cuda.nvtx.range_push(name)
        try:
            yield
        finally:
            torch.cuda.nvtx.range_pop()
    else:
        yield


# ---- names of the reference's module (`utils/profile.py:11-72`) ---------------------------------------------------
start_time = time.time()


class _ProfileView(dict):
    """Read-only `{name: {"calls": n, "total_time": s}}` view over the accumulated totals."""

    def _sync(self):
        dict.clear(self)
        for k, (n, t) in _totals.items():
            dict.__setitem__(self, k, {"calls": n, "total_time": t})
        return self

    def __getitem__(self, k):
        return dict.__getitem__(self._sync(), k)

    def __iter__(self):
        return dict.__iter__(self._sync())

    def __len__(self):
        return dict.__len__(self._sync())

    def items(self):
        return dict.items(self._sync())

    def keys(self):
        return dict.keys(self._sync())

    def __contains__(self, k):
        return k in _totals

    def __eq__(self, other):
        return dict(self._sync()) == other


profile_data = _ProfileView()


def profile_method(func):
    """Wrap one function with call counting and wall-clock accumulation."""
    global _enabled_print
    _enabled_print = True
    return _wrap_fn(func, f"{func.__module__}.{func.__qualname__}")


def print_profile_data():
    """Print the totals now (they are also printed at interpreter exit once anything was profiled)."""
    if _totals:
        print(f"Program cost {time.time() - start_time:.4f} seconds!")
        for name, (n, t) in _totals.items():
            print(f"{name}: {n} calls, {t:.4f} total seconds")
