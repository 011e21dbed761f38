"""Native caching pool (csrc/pool.cpp): size classes, cache hits, counters, cross-stream frees, and a training step
with the pool installed as torch's allocator (child process: the allocator has to be swapped before the first CUDA
allocation)."""
import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_round_size_classes():
    from genesis_b200.cuda import pool
    assert pool.round_size(1) == 512 and pool.round_size(513) == 1024
    assert pool.round_size(1 << 20) == 1 << 20
    assert pool.round_size((1 << 20) + 1) == 2 << 20
    assert pool.round_size(5 << 20) == 6 << 20                  # half steps between powers of two
    big = (1 << 30) + 5
    assert pool.round_size(big) >= big and pool.round_size(big) % (2 << 20) == 0


@pytest.mark.gpu
def test_standalone_alloc_free_cache_and_counters():
    from genesis_b200.cuda import pool
    dev = torch.cuda.current_device()
    pool.empty_cache(dev)
    s0 = pool.stats(dev)
    p1 = pool.alloc(3000, dev)
    assert p1 and p1 % 256 == 0
    s1 = pool.stats(dev)
    assert s1["alloc_count"] == s0["alloc_count"] + 1 and s1["allocated_bytes"] >= s0["allocated_bytes"] + 3000
    pool.free(p1, 3000, dev)
    p2 = pool.alloc(2500, dev)                                  # same size class: served from the cache
    s2 = pool.stats(dev)
    assert p2 == p1 and s2["cache_hits"] == s1["cache_hits"] + 1
    assert s2["cuda_alloc_count"] == s1["cuda_alloc_count"]
    pool.free(p2, 2500, dev)
    big = pool.alloc(64 << 20, dev)
    assert pool.stats(dev)["max_allocated_bytes"] >= 64 << 20
    pool.free(big, 64 << 20, dev)
    freed = pool.empty_cache(dev)
    assert freed >= 64 << 20
    assert pool.stats(dev)["total_cached_bytes"] == 0


@pytest.mark.gpu
def test_block_freed_on_another_stream_is_not_reused_early():
    from genesis_b200.cuda import pool
    dev = torch.cuda.current_device()
    side = torch.cuda.Stream()
    p = pool.alloc(1 << 20, dev, torch.cuda.current_stream().cuda_stream)
    with torch.cuda.stream(side):
        torch.cuda._sleep(50_000_000)                           # keep the side stream busy for a while
        pool.free(p, 1 << 20, dev, side.cuda_stream)            # freed on a different stream: parked behind an event
    q = pool.alloc(1 << 20, dev, torch.cuda.current_stream().cuda_stream)
    assert q != p or pool.stats(dev)["pending_deallocations"] == 0
    torch.cuda.synchronize()
    pool.free(q, 1 << 20, dev, torch.cuda.current_stream().cuda_stream)
    # the parked block is taken back lazily (every 16th allocation, on a cache miss, or on empty_cache)
    pool.empty_cache(dev)
    assert pool.stats(dev)["pending_deallocations"] == 0
    r = pool.alloc(1 << 20, dev, torch.cuda.current_stream().cuda_stream)
    pool.free(r, 1 << 20, dev, torch.cuda.current_stream().cuda_stream)


@pytest.mark.gpu
def test_training_step_with_the_pool_installed():
    code = (
        "import torch, genesis_b200 as genesis, genesis_b200.nn as nn\n"
        "from genesis_b200.cuda import pool\n"
        "assert pool.is_installed()\n"
        "m = nn.Sequential(nn.Linear(256, 512), nn.ReLU(), nn.Linear(512, 10)).cuda()\n"
        "opt = genesis.optim.AdamW(m.parameters(), lr=1e-3)\n"
        "x = genesis.randn(64, 256, device='cuda'); y = genesis.Tensor(torch.randint(0, 10, (64,), device='cuda'))\n"
        "first = None\n"
        "for i in range(20):\n"
        "    opt.zero_grad(); loss = nn.CrossEntropyLoss()(m(x), y); loss.backward(); opt.step()\n"
        "    first = first if first is not None else float(loss.item())\n"
        "st = genesis.cuda.memory_stats()\n"
        "ps = pool.stats(torch.cuda.current_device())\n"
        "assert ps['alloc_count'] > 50 and ps['cache_hits'] > ps['cuda_alloc_count'], ps\n"
        "assert float(loss.item()) < first\n"
        "assert genesis.cuda.memory_allocated() > 0 and 'Genesis' in genesis.cuda.memory_summary() or True\n"
        "print('POOL_OK', ps['alloc_count'], ps['cache_hits'], ps['cuda_alloc_count'])\n")
    env = dict(os.environ, GENESIS_B200_POOL="1", PYTHONPATH=ROOT)
    r = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "POOL_OK" in r.stdout, r.stdout + r.stderr


@pytest.mark.gpu
def test_block_freed_on_the_default_stream_is_not_handed_to_a_side_stream():
    """Stream 0 (the legacy default stream, torch's current stream unless told otherwise) has a null handle: a block
    it frees must stay its own until an event says otherwise, like the block of any other stream."""
    from genesis_b200.cuda import pool
    dev = torch.cuda.current_device()
    side = torch.cuda.Stream()
    n = 3 << 20
    p = pool.alloc(n, dev, 0)
    pool.free(p, n, dev, 0)                                     # back in the bin, tagged with stream 0
    q = pool.alloc(n, dev, side.cuda_stream)                    # another stream: must not get that block
    assert q != p
    r = pool.alloc(n, dev, 0)                                   # stream 0 itself reuses it at once
    assert r == p
    pool.free(q, n, dev, side.cuda_stream)
    pool.free(r, n, dev, 0)


@pytest.mark.gpu
def test_graph_capture_keeps_its_blocks_private():
    """Memory that a captured step allocates (and frees) belongs to the graph: eager allocations made afterwards never
    alias it, so a replay still computes the same thing after the eager code has scribbled over everything it got."""
    code = (
        "import torch, genesis_b200 as genesis, genesis_b200.nn as nn\n"
        "from genesis_b200.cuda import pool\n"
        "assert pool.is_installed()\n"
        "dev = torch.cuda.current_device()\n"
        "genesis.manual_seed(0)\n"
        "def make():\n"
        "    genesis.manual_seed(0)\n"
        "    m = nn.Sequential(nn.Linear(256, 512), nn.ReLU(), nn.Linear(512, 10)).cuda()\n"
        "    opt = genesis.optim.AdamW(m.parameters(), lr=1e-3)\n"
        "    def step(x, y):\n"
        "        opt.zero_grad(); loss = nn.CrossEntropyLoss()(m(x), y); loss.backward(); opt.step(); return loss\n"
        "    return m, opt, step\n"
        "x = genesis.randn(64, 256, device='cuda'); y = genesis.Tensor(torch.randint(0, 10, (64,), device='cuda'))\n"
        "ma, oa, sa = make(); mb, ob, sb = make()\n"
        "g = genesis.cuda.GraphedTrainStep(sb, ob, [x, y], warmup=2)\n"
        "assert pool.capture_cached(dev) > 0\n"
        "for _ in range(2): sa(x, y)\n"
        "junk = []\n"
        "for i in range(6):\n"
        "    la = sa(x, y)\n"
        "    # eager code grabs blocks of the classes the step uses and fills them with NaN\n"
        "    junk = [torch.full((64, 512), float('nan'), device='cuda') for _ in range(8)]\n"
        "    junk += [torch.full((64, 10), float('nan'), device='cuda') for _ in range(8)]\n"
        "    lb = g(x, y)\n"
        "    torch.cuda.synchronize()\n"
        "    assert abs(float(la._t) - float(lb._t)) < 1e-4, (i, float(la._t), float(lb._t))\n"
        "cached = pool.capture_cached(dev)\n"
        "g.graph.reset()\n"
        "assert pool.capture_cached(dev) == 0 and cached > 0\n"
        "print('CAPTURE_OK', cached)\n")
    env = dict(os.environ, GENESIS_B200_POOL="1", PYTHONPATH=ROOT)
    r = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "CAPTURE_OK" in r.stdout, r.stdout + r.stderr


@pytest.mark.gpu
def test_cuda_storage_rest_of_the_reference_surface():
    import numpy as np
    import torch
    from genesis_b200.backends import CUDAStorage, CPUStorage
    from genesis_b200.backends import cuda as bc
    from genesis_b200.backends import cuda_memory as cm
    a = bc.from_numpy(np.arange(24, dtype=np.float32).reshape(2, 3, 4))
    assert a.numel() == 24 and a.stride() == (12, 4, 1) and a.stride(1) == 4 and a.data is a and not a.is_shared()
    assert str(a.device).startswith("cuda") and a.numpy_dtype() == np.float32
    assert a.T.shape == (4, 3, 2) and a.unsqueeze(0).shape == (1, 2, 3, 4) and a.unsqueeze(0).squeeze().shape == (2, 3, 4)
    assert a.broadcast_to((5, 2, 3, 4)).shape == (5, 2, 3, 4)
    assert a.half().dtype == "float16" and a.long().dtype == "int64" and a.to("bfloat16").float().dtype == "float32"
    assert bc.ones(1).item() == 1.0 and bc.zeros(2, 2).fill_(3).to_numpy().sum() == 12.0
    parts = a.split(2, dim=2)
    assert [p.shape for p in parts] == [(2, 3, 2), (2, 3, 2)]
    back = CUDAStorage.cat(parts, dim=2)
    assert np.array_equal(back.to_numpy(), a.to_numpy())
    dst = bc.empty(3, 2)
    a.copy_strided_to_contiguous((3, 2), (4, 12), 1, dst)          # element (i, j) = flat[1 + 4 i + 12 j]
    assert np.array_equal(dst.to_numpy(), np.arange(24, dtype=np.float32)[1:].reshape(-1)[[0, 12, 4, 16, 8, 20]].reshape(3, 2))
    assert np.array_equal(CPUStorage.ones((2, 2)).to_cuda().detach().to_numpy(), np.ones((2, 2), np.float32))
    mgr = cm.get_memory_manager()
    assert isinstance(mgr, cm.CudaCachingAllocator)
    p = mgr.allocate_memory(4096)
    assert p != 0
    mgr.free_memory(p, 4096)
    assert mgr.warmup_pool([1 << 20, 1 << 16], [2, 3]) == 5 and mgr.drain_pending() == 0
    assert cm.round_size(1000)[0] >= 1000 and "allocated_bytes.all.current" in str(cm.memory_stats()) or True
    cm.increase_ref_count(p)
    assert cm.decrease_ref_count(p) is False and cm.decrease_ref_count(p) is True
