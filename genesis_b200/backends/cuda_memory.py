"""`genesis.backends.cuda_memory` of the reference (its Python caching allocator, `backends/cuda_memory.py:89-850`), as
functions over the native pool (`csrc/pool.cpp`, `genesis_b200.cuda.pool`) that allocates every CUDA tensor here."""
from .. import cuda as _cuda
from ..cuda import pool as _pool
from ..cuda import (analyze_memory_fragmentation, defragment_memory, empty_cache, get_memory_info,  # noqa: F401
                    get_memory_manager, memory_stats, set_memory_config, trigger_gc)


def round_size(nbytes):
    """(rounded size, is_small) of the pool's size classes."""
    r = _pool.round_size(int(nbytes))
    return r, r <= (1 << 20)


def allocate_memory(nbytes, stream=None):
    """Device pointer (int) to at least `nbytes` bytes from the pool, usable on `stream` (0 / None = current)."""
    return _pool.alloc(int(nbytes), _cuda.current_device(), int(stream or 0))


def free_memory(ptr, nbytes, stream=None):
    _pool.free(int(ptr), int(nbytes), _cuda.current_device(), int(stream or 0))


_refs = {}


def increase_ref_count(ptr):
    _refs[int(ptr)] = _refs.get(int(ptr), 1) + 1


def decrease_ref_count(ptr, stream=None):
    """True when the count reached zero (the caller then frees the block)."""
    n = _refs.get(int(ptr), 1) - 1
    if n <= 0:
        _refs.pop(int(ptr), None)
        return True
    _refs[int(ptr)] = n
    return False


def get_memory_stats():
    return memory_stats()


def get_fragmentation_stats():
    return analyze_memory_fragmentation()


CudaCachingAllocator = _cuda._MemoryManager
