"""Python face of the native caching pool (`csrc/pool.cpp`).

The pool is a size-class caching allocator over `cudaMalloc` (small classes 512 B .. 1 MB,
large classes 2 MB .. 1 GB in 2 MB-rounded power-of-two/half steps, direct allocation
above), stream-aware (a block freed on another stream than it was allocated on is parked
behind a CUDA event), with always-on counters.  It exports the two C entry points torch's
`CUDAPluggableAllocator` expects, so `install()` routes every torch CUDA allocation through
it; it can also be used standalone (`alloc` / `free`) for communication buffers.  It is installed by default when the
package is imported on a machine with a GPU (`GENESIS_B200_POOL=0` keeps torch's allocator), and it is aware of
CUDA graph captures made through `genesis_b200.cuda.graph` (`begin_capture` / `end_capture` / `release_capture`).
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
        lib.gb_pool_begin_capture.argtypes = [ctypes.c_int]
        lib.gb_pool_begin_capture.restype = ctypes.c_int
        lib.gb_pool_end_capture.argtypes = [ctypes.c_int]
        lib.gb_pool_end_capture.restype = None
        lib.gb_pool_release_capture.argtypes = [ctypes.c_int, ctypes.c_int]
        lib.gb_pool_release_capture.restype = ctypes.c_int64
        lib.gb_pool_capture_cached.argtypes = [ctypes.c_int]
        lib.gb_pool_capture_cached.restype = ctypes.c_int64
        lib._pool_bound = True
    return lib


def install(strict=True):
    """Make the pool torch's CUDA allocator.  Must run before the first CUDA allocation of the process: torch refuses
    to swap an allocator that is already in use (then this raises, or returns False when `strict` is off)."""
    global _installed
    if _installed:
        return True
    _L()
    try:
        alloc = torch.cuda.memory.CUDAPluggableAllocator(_lib.LIB_PATH, "gb_pool_alloc", "gb_pool_free")
        torch.cuda.memory.change_current_allocator(alloc)
    except RuntimeError:
        if strict:
            raise
        return False
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


def begin_capture(device=0):
    """A CUDA graph capture starts on `device`: blocks handed out from now on belong to it (see csrc/pool.cpp).
    Returns the capture id (0: the pool is not in use, or a capture is already open)."""
    if not (_installed or _standalone):
        return 0
    return int(_L().gb_pool_begin_capture(device))


def end_capture(device=0):
    if _installed or _standalone:
        _L().gb_pool_end_capture(device)


def release_capture(device, capture_id):
    """The graph is destroyed: its private blocks return to the common bins."""
    if capture_id and (_installed or _standalone):
        return int(_L().gb_pool_release_capture(device, capture_id))
    return 0


def capture_cached(device=0):
    return int(_L().gb_pool_capture_cached(device)) if (_installed or _standalone) else 0


def round_size(nbytes):
    return int(_L().gb_pool_round_size(nbytes))


# The pool is the allocator of every CUDA tensor unless GENESIS_B200_POOL=0 asks for torch's own.  A process that
# made CUDA allocations before importing this package keeps torch's allocator (it cannot be swapped any more);
# GENESIS_B200_POOL=1 turns that case into an error instead.
_mode = os.environ.get("GENESIS_B200_POOL", "auto")
if _mode != "0" and torch.cuda.is_available() and _lib.available():
    install(strict=(_mode == "1"))
