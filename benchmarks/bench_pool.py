"""Allocator benchmark: the native caching pool (csrc/pool.cpp) installed as torch's allocator against torch's own
caching allocator, on the allocation patterns the reference reports (same-size allocations, > 1 MB allocations, a
transformer-like pattern, allocation under memory pressure).

    python benchmarks/bench_pool.py            # runs both arms in child processes and prints one JSON line per pattern

Each arm runs in a fresh process because an allocator can only be swapped before the first CUDA allocation.
Times are host wall-clock per allocate-and-free pair (the cost the allocator adds to an op), after warm-up.
Reference counterpart: benchmark/bench_cuda_storage.py and docs/en/memory-allocator-optimization.md.
"""
import json
import os
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

PATTERNS = {
    # name: list of byte sizes allocated in order and freed in reverse order, per iteration
    "same_size_4KB": [4096] * 64,
    "same_size_4MB": [4 << 20] * 16,
    "large_1MB_to_256MB": [1 << 20, 8 << 20, 64 << 20, 256 << 20, 32 << 20, 2 << 20],
    "transformer_like": [8 * 2048 * 896 * 2, 8 * 2048 * 4864 * 2, 8 * 2048 * 4864 * 2, 8 * 2048 * 896 * 2,
                         8 * 14 * 2048 * 4, 8 * 2048 * 896 * 2, 8 * 2048 * 128 * 2, 8 * 2048 * 128 * 2] * 4,
}


def child():
    import torch
    sys.path.insert(0, ROOT)
    import genesis_b200  # noqa: F401  (installs the pool when GENESIS_B200_POOL=1)
    from genesis_b200.cuda import pool
    arm = "pool" if pool.is_installed() else "torch"
    out = {}
    for name, sizes in PATTERNS.items():
        def once():
            ts = [torch.empty(n, dtype=torch.uint8, device="cuda") for n in sizes]
            del ts
        for _ in range(20):
            once()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        iters = 200
        for _ in range(iters):
            once()
        torch.cuda.synchronize()
        out[name] = (time.perf_counter() - t0) / (iters * len(sizes)) * 1e6
    # memory pressure: hold 60% of the free memory, then churn 64 MB blocks
    free, _total = torch.cuda.mem_get_info()
    hog = torch.empty(int(free * 0.6), dtype=torch.uint8, device="cuda")
    def churn():
        ts = [torch.empty(64 << 20, dtype=torch.uint8, device="cuda") for _ in range(8)]
        del ts
    for _ in range(10):
        churn()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(100):
        churn()
    torch.cuda.synchronize()
    out["memory_pressure_64MB"] = (time.perf_counter() - t0) / 800 * 1e6
    del hog
    print(json.dumps({"arm": arm, "us_per_alloc_free": out}), flush=True)


def main():
    if os.environ.get("GB_POOL_BENCH_CHILD") == "1":
        child()
        return
    res = {}
    for arm, flag in (("torch", "0"), ("pool", "1")):
        env = dict(os.environ, GB_POOL_BENCH_CHILD="1", GENESIS_B200_POOL=flag)
        r = subprocess.run([sys.executable, os.path.abspath(__file__)], env=env, capture_output=True, text=True, timeout=600)
        line = [l for l in r.stdout.splitlines() if l.startswith("{")]
        if r.returncode != 0 or not line:
            print(json.dumps({"arm": arm, "error": (r.stderr or r.stdout)[-400:]}))
            continue
        res[arm] = json.loads(line[-1])["us_per_alloc_free"]
    if "torch" in res and "pool" in res:
        for k in res["torch"]:
            print(json.dumps({"pattern": k, "torch_us": res["torch"][k], "pool_us": res["pool"][k],
                              "pool_speedup": res["torch"][k] / res["pool"][k]}))


if __name__ == "__main__":
    main()
