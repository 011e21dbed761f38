"""`genesis_b200.cuda`: device management and memory-pool statistics.

Parity: reference `genesis/cuda/__init__.py:64-420` (function names, the nested
`memory_stats()` dict, the `memory_summary()` section headers, `empty_cache()` return
dict, `GENESIS_CUDA_ALLOC_CONF` parsing) and `genesis/backends/cuda_memory.py:536-576`
(flat allocator statistics).  The pool itself is the native size-class caching
allocator in `csrc/pool.cpp` (`genesis_b200.cuda.pool`); when it is installed as
torch's CUDA allocator every tensor allocation goes through it and the numbers below
are its counters, otherwise they are derived from torch's caching allocator.
"""
import logging
import os

import torch

from . import pool
from .. import amp  # `from genesis.cuda import amp` is the spelling of the reference's README

logger = logging.getLogger(__name__)

_config = {}
_memory_fraction = 1.0


# ---- devices ----------------------------------------------------------------------
def is_available():
    return torch.cuda.is_available()


def device_count():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def current_device():
    return torch.cuda.current_device() if torch.cuda.is_available() else 0


def set_device(device):
    if hasattr(device, "index"):
        device = device.index or 0
    if not torch.cuda.is_available():
        raise RuntimeError("CUDA is not available")
    if device < 0 or device >= torch.cuda.device_count():
        raise RuntimeError(f"Invalid device id: {device}")
    torch.cuda.set_device(device)


def get_device_name(device=None):
    return torch.cuda.get_device_name(device) if torch.cuda.is_available() else "cpu"


def get_device_capability(device=None):
    return torch.cuda.get_device_capability(device) if torch.cuda.is_available() else (0, 0)


def synchronize(device=None):
    if torch.cuda.is_available():
        torch.cuda.synchronize(device)


def current_stream(device=None):
    return torch.cuda.current_stream(device)


Stream = torch.cuda.Stream
Event = torch.cuda.Event
stream = torch.cuda.stream


# ---- memory info --------------------------------------------------------------------
def get_memory_info(device=None):
    if not torch.cuda.is_available():
        return {"gpu_memory": {"error": "CUDA not available"}}
    free, total = torch.cuda.mem_get_info(device)
    used = total - free
    mb = 1024.0 * 1024.0
    return {"gpu_memory": {"total_mb": total / mb, "used_mb": used / mb, "free_mb": free / mb,
                           "usage_ratio": f"{used / max(total, 1):.2%}"}}


def _flat_stats(device=None):
    """Allocator statistics in the reference's flat layout (`cuda_memory.py:536-576`)."""
    thr = float(os.environ.get("GENESIS_MEMORY_PRESSURE_THRESHOLD", 0.9))
    crit = float(os.environ.get("GENESIS_MEMORY_CRITICAL_THRESHOLD", 0.95))
    pressure = 0.0
    if torch.cuda.is_available():
        free, total = torch.cuda.mem_get_info(device)
        pressure = 1.0 - free / max(total, 1)
    if pool.is_installed() or pool.standalone_used():
        s = pool.stats(device if device is not None else current_device())
    elif torch.cuda.is_available():
        ts = torch.cuda.memory_stats(device)
        allocs = ts.get("allocation.all.allocated", 0)
        seg = ts.get("segment.all.allocated", 0)
        s = {
            "alloc_count": allocs, "free_count": ts.get("allocation.all.freed", 0),
            "cache_hits": max(allocs - seg, 0), "cuda_alloc_count": seg,
            "small_pool_blocks": ts.get("inactive_split.small_pool.current", 0),
            "large_pool_blocks": ts.get("inactive_split.large_pool.current", 0),
            "small_pool_bytes": ts.get("inactive_split_bytes.small_pool.current", 0),
            "large_pool_bytes": ts.get("inactive_split_bytes.large_pool.current", 0),
            "total_cached_bytes": ts.get("reserved_bytes.all.current", 0) - ts.get("allocated_bytes.all.current", 0),
            "pending_deallocations": 0, "pending_checks": 0,
            "allocated_bytes": ts.get("allocated_bytes.all.current", 0),
            "max_allocated_bytes": ts.get("allocated_bytes.all.peak", 0),
            "reserved_bytes": ts.get("reserved_bytes.all.current", 0),
            "max_reserved_bytes": ts.get("reserved_bytes.all.peak", 0),
        }
    else:
        s = {k: 0 for k in ("alloc_count", "free_count", "cache_hits", "cuda_alloc_count", "small_pool_blocks",
                            "large_pool_blocks", "small_pool_bytes", "large_pool_bytes", "total_cached_bytes",
                            "pending_deallocations", "pending_checks", "allocated_bytes", "max_allocated_bytes",
                            "reserved_bytes", "max_reserved_bytes")}
    s["cache_hit_rate"] = s["cache_hits"] / s["alloc_count"] if s["alloc_count"] else 0.0
    s["memory_pressure"] = pressure
    s["memory_pressure_threshold"] = thr
    s["memory_critical_threshold"] = crit
    return s


get_memory_stats = _flat_stats


def memory_stats(device=None):
    s = _flat_stats(device)
    blocks = s["small_pool_blocks"] + s["large_pool_blocks"]
    mb = 1024.0 * 1024.0
    return {
        "allocation": {"total_allocations": s["alloc_count"], "active_blocks": blocks,
                       "current_active_memory_mb": s["total_cached_bytes"] / mb,
                       "allocated_mb": s["allocated_bytes"] / mb, "reserved_mb": s["reserved_bytes"] / mb},
        "cache": {"pool_hits": s["cache_hits"], "pool_misses": s["alloc_count"] - s["cache_hits"],
                  "hit_rate": s["cache_hit_rate"], "pool_blocks": blocks,
                  "pool_size_mb": s["total_cached_bytes"] / mb, "ref_count_saves": 0},
        "pressure": {"memory_pressure": s["memory_pressure"],
                     "critical_pressure": s["memory_pressure"] > s["memory_critical_threshold"],
                     "pressure_cleanups": 0, "critical_cleanups": 0,
                     "pressure_threshold": s["memory_pressure_threshold"],
                     "critical_threshold": s["memory_critical_threshold"]},
        "fragmentation": {"overall_fragmentation": 0.0, "pool_fragmentation": 0.0, "defrag_operations": 0,
                          "fragmentation_threshold": 0.3, "trend": "stable",
                          "recommendation": "No action needed - size-class pool does not fragment"},
        "memory_info": get_memory_info(device),
    }


def memory_summary(device=None):
    st = memory_stats(device)
    a, c, p, f, mi = st["allocation"], st["cache"], st["pressure"], st["fragmentation"], st["memory_info"]
    lines = [
        "=" * 60, "Genesis CUDA Memory Summary", "=" * 60, "",
        "ALLOCATION:",
        f'  Total allocations: {a["total_allocations"]:,}',
        f'  Active blocks: {a["active_blocks"]:,}',
        f'  Current memory: {a["current_active_memory_mb"]:.2f} MB', "",
        "CACHE PERFORMANCE:",
        f'  Pool hits: {c["pool_hits"]:,}',
        f'  Pool misses: {c["pool_misses"]:,}',
        f'  Hit rate: {c["hit_rate"]:.2%}',
        f'  Pool blocks: {c["pool_blocks"]:,}',
        f'  Pool size: {c["pool_size_mb"]:.2f} MB',
        f'  Reference count saves: {c["ref_count_saves"]:,}', "",
        "MEMORY PRESSURE:",
        f'  Current pressure: {p["memory_pressure"]:.2%}',
        f'  Critical pressure: {"Yes" if p["critical_pressure"] else "No"}',
        f'  Pressure cleanups: {p["pressure_cleanups"]:,}',
        f'  Critical cleanups: {p["critical_cleanups"]:,}',
        f'  Pressure threshold: {p["pressure_threshold"]:.2%}', "",
        "FRAGMENTATION:",
        f'  Overall fragmentation: {f["overall_fragmentation"]:.3f}',
        f'  Pool fragmentation: {f["pool_fragmentation"]:.3f}',
        f'  Defrag operations: {f["defrag_operations"]:,}',
        f'  Fragmentation trend: {f["trend"]}',
        f'  Recommendation: {f["recommendation"]}',
    ]
    gm = mi.get("gpu_memory", {})
    if gm and "error" not in gm:
        lines += ["", "GPU MEMORY:", f'  Total: {gm["total_mb"]:.1f} MB', f'  Used: {gm["used_mb"]:.1f} MB',
                  f'  Free: {gm["free_mb"]:.1f} MB', f'  Usage: {gm["usage_ratio"]}']
    lines += ["", "RECOMMENDATIONS:"]
    if p["critical_pressure"]:
        lines.append("  Memory pressure is critical: call empty_cache() or reduce the batch size")
    elif c["hit_rate"] < 0.5 and a["total_allocations"] > 100:
        lines.append("  Low pool hit rate: allocation sizes vary a lot between steps")
    else:
        lines.append("  Memory usage looks healthy")
    lines.append("=" * 60)
    return "\n".join(lines)


def empty_cache():
    before = _flat_stats()
    if pool.is_installed() or pool.standalone_used():
        pool.empty_cache(current_device())
    if torch.cuda.is_available():
        torch.cuda.empty_cache()
    after = _flat_stats()
    return {
        "freed_memory_mb": (before["total_cached_bytes"] - after["total_cached_bytes"]) / (1024.0 * 1024.0),
        "cleared_pools": (before["small_pool_blocks"] + before["large_pool_blocks"])
        - (after["small_pool_blocks"] + after["large_pool_blocks"]),
        "defragmentation_performed": False,
        "stats": {"before": before, "after": after},
    }


def trigger_gc():
    import gc
    gc.collect()
    return empty_cache()


def memory_allocated(device=None):
    return _flat_stats(device)["allocated_bytes"]


def memory_reserved(device=None):
    return _flat_stats(device)["reserved_bytes"]


memory_cached = memory_reserved


def max_memory_allocated(device=None):
    return _flat_stats(device)["max_allocated_bytes"]


def max_memory_reserved(device=None):
    return _flat_stats(device)["max_reserved_bytes"]


max_memory_cached = max_memory_reserved


def reset_max_memory_allocated(device=None):
    if pool.is_installed() or pool.standalone_used():
        pool.reset_peak(device if device is not None else current_device())
    elif torch.cuda.is_available():
        torch.cuda.reset_peak_memory_stats(device)


reset_max_memory_cached = reset_max_memory_allocated
reset_memory_stats = reset_max_memory_allocated


def set_memory_fraction(fraction, device=None):
    """Cap the pool at `fraction` of the device memory."""
    global _memory_fraction
    if not 0.0 < fraction <= 1.0:
        raise ValueError("fraction must be in (0, 1]")
    _memory_fraction = fraction
    if torch.cuda.is_available():
        if pool.is_installed():
            _, total = torch.cuda.mem_get_info(device)
            pool.set_limit(device if device is not None else current_device(), int(total * fraction))
        else:
            torch.cuda.set_per_process_memory_fraction(fraction, device)


# ---- GENESIS_CUDA_ALLOC_CONF="k=v,k=v" ------------------------------------------------
def _parse_memory_config(text=None):
    text = os.environ.get("GENESIS_CUDA_ALLOC_CONF", "") if text is None else text
    cfg = {}
    for item in text.split(","):
        item = item.strip()
        if not item or "=" not in item:
            continue
        k, v = (x.strip() for x in item.split("=", 1))
        lv = v.lower()
        if lv in ("true", "false"):
            cfg[k] = lv == "true"
        else:
            try:
                cfg[k] = int(v)
            except ValueError:
                try:
                    cfg[k] = float(v)
                except ValueError:
                    cfg[k] = v
    return cfg


def apply_memory_config():
    global _config
    _config = _parse_memory_config()
    if "memory_fraction" in _config and torch.cuda.is_available():
        set_memory_fraction(float(_config["memory_fraction"]))
    return _config


def set_memory_config(config):
    _config.update(config)


def get_memory_config():
    return dict(_config)


def defragment_memory():
    return empty_cache()


def analyze_memory_fragmentation():
    return memory_stats()["fragmentation"]


get_fragmentation_stats = analyze_memory_fragmentation

_config = _parse_memory_config()


class _MemoryManager:
    """Handle on the allocator statistics of one device (the reference returns its Python pool object here,
    `cuda/__init__.py`; this one reads the native pool's counters or torch's allocator)."""

    def __init__(self, device):
        self.device = device

    def get_stats(self):
        return memory_stats(self.device)

    def empty_cache(self):
        return empty_cache()

    def memory_summary(self):
        return memory_summary(self.device)

    # ---- the reference allocator's method names (`backends/cuda_memory.py:165-600`) over the native pool ----
    def memory_stats(self):
        return memory_stats(self.device)

    def trigger_gc(self):
        return trigger_gc()

    def allocate_memory(self, nbytes, stream=None):
        from . import pool
        return pool.alloc(int(nbytes), int(self.device), int(stream or 0))

    def free_memory(self, ptr, nbytes, stream=None):
        from . import pool
        pool.free(int(ptr), int(nbytes), int(self.device), int(stream or 0))

    def increase_ref_count(self, ptr):
        from ..backends import cuda_memory
        cuda_memory.increase_ref_count(ptr)

    def decrease_ref_count(self, ptr, stream=None):
        from ..backends import cuda_memory
        return cuda_memory.decrease_ref_count(ptr, stream)

    def drain_pending(self, max_events=None):
        """Blocks freed on another stream become reusable once their event has completed; the native pool polls those
        events on every allocation, so there is nothing to drain by hand.  Returns 0."""
        return 0

    def warmup_pool(self, sizes=(), counts=None):
        """Pre-populates the pool's free lists: allocates and frees `counts[i]` (default 1) blocks of `sizes[i]` bytes."""
        from . import pool
        n = 0
        for i, sz in enumerate(sizes):
            c = 1 if counts is None else int(counts[i])
            ptrs = [pool.alloc(int(sz), int(self.device), 0) for _ in range(c)]
            for p in ptrs:
                pool.free(p, int(sz), int(self.device), 0)
            n += c
        return n


def get_memory_manager(device=None):
    return _MemoryManager(current_device() if device is None else device)


from ..device import Device  # noqa: E402,F401  (re-exported as in the reference)

from .graphs import CUDAGraph, GraphedCallable, GraphedTrainStep, graph, make_graphed_callable  # noqa: E402,F401
