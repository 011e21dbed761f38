"""`genesis.cuda` interface without a GPU: dictionary keys, summary section names, allocator configuration parsing
(the reference's tests check exactly these surfaces: tests/test_cuda_interface.py, tests/test_cuda_memory_management.py)."""
import os

import genesis_b200 as genesis


def test_memory_stats_keys_and_summary_sections():
    c = genesis.cuda
    st = c.memory_stats()
    assert set(st.keys()) >= {"allocation", "cache", "fragmentation", "memory_info", "pressure"}
    text = c.memory_summary()
    for header in ("Genesis CUDA Memory Summary", "ALLOCATION:", "CACHE PERFORMANCE:", "MEMORY PRESSURE:", "FRAGMENTATION:"):
        assert header in text, header
    flat = c.get_memory_stats()
    assert isinstance(flat, dict)
    assert c.memory_allocated() >= 0 and c.memory_reserved() >= 0
    assert c.max_memory_allocated() >= 0 and c.max_memory_reserved() >= 0
    c.reset_max_memory_allocated()
    c.empty_cache()
    c.trigger_gc()
    assert isinstance(c.get_memory_info(), dict)
    assert isinstance(c.analyze_memory_fragmentation(), dict)
    c.defragment_memory()


def test_allocator_config_parsing(monkeypatch):
    c = genesis.cuda
    assert c._parse_memory_config("garbage_collection_threshold=0.7,max_split_size_mb=128") == {
        "garbage_collection_threshold": 0.7, "max_split_size_mb": 128}
    assert c._parse_memory_config("") == {}
    monkeypatch.setenv("GENESIS_CUDA_ALLOC_CONF", "max_split_size_mb=64, expandable_segments=True")
    cfg = c._parse_memory_config()
    assert cfg["max_split_size_mb"] == 64 and cfg["expandable_segments"] in (True, "True")
    c.set_memory_config({"max_split_size_mb": 32})
    assert c.get_memory_config()["max_split_size_mb"] == 32


def test_device_queries_without_a_gpu_do_not_raise():
    c = genesis.cuda
    if c.is_available():
        assert c.device_count() >= 1 and isinstance(c.get_device_name(), str)
    else:
        assert c.device_count() == 0
    d = genesis.device("cpu")
    assert str(d) == "cpu" or "cpu" in repr(d)
    x = genesis.randn(2, 3)
    assert x.device == d or "cpu" in str(x.device)


def test_ctypes_signatures_match_the_c_prototypes():
    """Every binding in ops/native.py has the argument list of its `extern "C"` prototype (checked from the sources,
    no GPU needed)."""
    from genesis_b200.ops import abi_check
    assert abi_check.mismatches() == []
