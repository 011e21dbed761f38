"""Python face of the native caching pool (`csrc/pool.cpp`).

The pool is a size-class caching allocator over `cudaMalloc` (small classes 512 B .. 1 MB,
large classes 2 MB .. 1 GB in 2 MB-rounded power-of-two/half steps, direct allocation
above), stream-aware (a block freed on another stream than it was allocated on is parked
behind a CUDA event), with always-on counters.  It exports the two C entry points torch's
`CUDAPluggableAllocator` expects, so `install()` routes every torch CUDA allocation through
it; it can also be used standalone (`alloc` / `free`) for communication buffers.
Reference counterpart: `genesis/backends/cuda_memory.py:111-576`.
"""
import ctypes
import os

import torch

from .. import _lib

_installed = False
_standalone = False
_NSTAT = 16
_STAT_NAMES = ("alloc_count", "free_count", "cache_hits", "cuda_alloc_count", "small_pool_blocks",
               "large_pool_blocks", "small_pool_bytes", "large_pool_bytes", "total_cached_bytes",
               "pending_deallocations", "pending_checks", "allocated_bytes", "max_allocated_bytes",
               "reserved_bytes", "max_reserved_bytes", "oom_retries")


def _L():
    lib = _lib.get(required=True)
    if not getattr(lib, "_pool_bound", False):
        lib.gb_pool_alloc.restype = ctypes.c_void_p
        lib.gb_pool_alloc.argtypes = [ctypes.c_ssize_t, ctypes.c_int, ctypes.c_void_p]
        lib.gb_pool_free.restype = None
        lib.gb_pool_free.argtypes = [ctypes.c_void_p, ctypes.c_ssize_t, ctypes.c_int, ctypes.c_void_p]
        lib.gb_pool_stats.argtypes = [ctypes.c_int, ctypes.POINTER(ctypes.c_int64)]
        lib.gb_pool_empty_cache.argtypes = [ctypes.c_int]
        lib.gb_pool_empty_cache.restype = ctypes.c_int64
        lib.gb_pool_reset_peak.argtypes = [ctypes.c_int]
        lib.gb_pool_set_limit.argtypes = [ctypes.c_int, ctypes.c_int64]
        lib.gb_pool_round_size.argtypes = [ctypes.c_int64]
        lib.gb_pool_round_size.restype = ctypes.c_int64
        lib._pool_bound = True
    return lib


def install():
    """Make the pool torch's CUDA allocator. Must run before the first CUDA allocation."""
    global _installed
    if _installed:
        return True
    _L()
    alloc = torch.cuda.memory.CUDAPluggableAllocator(_lib.LIB_PATH, "gb_pool_alloc", "gb_pool_free")
    torch.cuda.memory.change_current_allocator(alloc)
    _installed = True
    return True


def is_installed():
    return _installed


def standalone_used():
    return _standalone


def alloc(nbytes, device=0, stream=0):
    global _standalone
    _standalone = True
    return _L().gb_pool_alloc(nbytes, device, ctypes.c_void_p(stream))


def free(ptr, nbytes, device=0, stream=0):
    _L().gb_pool_free(ctypes.c_void_p(ptr), nbytes, device, ctypes.c_void_p(stream))


def stats(device=0):
    buf = (ctypes.c_int64 * _NSTAT)()
    _L().gb_pool_stats(device, buf)
    return {k: int(buf[i]) for i, k in enumerate(_STAT_NAMES)}


def empty_cache(device=0):
    return int(_L().gb_pool_empty_cache(device))


def reset_peak(device=0):
    _L().gb_pool_reset_peak(device)


def set_limit(device, nbytes):
    _L().gb_pool_set_limit(device, nbytes)


def round_size(nbytes):
    return int(_L().gb_pool_round_size(nbytes))


if os.environ.get("GENESIS_B200_POOL", "0") == "1" and torch.cuda.is_available():
    install()
