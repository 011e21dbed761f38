"""`genesis.amp.amp_cache` of the reference (`amp/amp_cache.py:14-145`): a per-region cache of parameter casts with hit
/ miss counters.  Here the cache that autocast actually uses lives in `amp_state.cache` (thread-local, keyed by tensor
identity and version, cleared when an autocast region is entered) and `function.cast` consults it; this class is the
reference's interface over the same store."""
from ..amp_state import amp_state
from ..function import cast as _cast


class AMPCache:
    def __init__(self):
        self.enabled = True
        self.hits = 0
        self.misses = 0

    def cached_cast(self, tensor, target_dtype):
        """`tensor` in `target_dtype` (a genesis dtype, name or torch dtype); repeated casts of the same unchanged
        parameter inside one autocast region return the cached tensor."""
        from ..dtypes import get_dtype
        td = get_dtype(target_dtype).torch_dtype
        if tensor._t.dtype == td:
            return tensor
        key = (id(tensor), td)
        hit = amp_state.cache.get(key) if self.enabled else None
        if hit is not None and hit[0] is tensor and hit[2] == tensor._version:
            self.hits += 1
            return hit[1]
        self.misses += 1
        out = _cast(tensor, td)
        if self.enabled and key not in amp_state.cache:
            amp_state.cache[key] = (tensor, out, tensor._version)
        return out

    def clear(self):
        amp_state.cache.clear()

    def set_enabled(self, enabled: bool):
        self.enabled = bool(enabled)
        if not self.enabled:
            self.clear()

    def get_stats(self):
        total = self.hits + self.misses
        return {"hits": self.hits, "misses": self.misses, "size": len(amp_state.cache),
                "hit_rate": (self.hits / total) if total else 0.0}

    def reset_stats(self):
        self.hits = self.misses = 0


_cache = None


def get_amp_cache() -> AMPCache:
    global _cache
    if _cache is None:
        _cache = AMPCache()
    return _cache
