"""All-reduce sweep (BASELINE config 5, row C1): the fused peer-memory kernel against NCCL, 1 KB - 1 GB.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29533 \
        benchmarks/bench_allreduce.py [--max-mb 1024] [--ctas 32]

Device time from CUDA events, max over ranks.  Roofline of a two-shot all-reduce of S bytes on N GPUs:
t = 2 (N-1)/N S / link bandwidth, reported against the nominal 900 GB/s per direction and against the measured
peer-copy bandwidth of 770 GB/s.  Three columns per size: the fused fp32 kernel (in place over a symmetric buffer), the
16-bit-wire kernel (fp32 bucket in local memory, bf16 values on NVLink, pack and cast inside the kernel; its bus
bandwidth is quoted for the fp32 bytes it reduces), and `torch.distributed.all_reduce` over NCCL with NCCL's own
defaults (NVLS as NCCL chooses).  Rank 0 prints one JSON line per size.
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as tdist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import genesis_b200  # noqa: E402,F401
from genesis_b200 import distributed as dist  # noqa: E402
from genesis_b200.distributed import symm  # noqa: E402
from genesis_b200.ops import native as N  # noqa: E402

LINK_GBS = 770.0
NOMINAL_GBS = 900.0


def timed(fn, iters, world):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    tdist.barrier()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    t = torch.tensor([a.elapsed_time(b) / iters], device="cuda", dtype=torch.float64)
    tdist.all_reduce(t, op=tdist.ReduceOp.MAX)
    return float(t.item())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--max-mb", type=int, default=1024)
    ap.add_argument("--ctas", type=int, default=0, help="0 = automatic")
    ap.add_argument("--dtype", default="float32")
    ap.add_argument("--quick", action="store_true", help="eight sizes instead of every power of two")
    a = ap.parse_args()
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
    dist.init_process_group("nccl")
    rank, world = dist.get_rank(), dist.get_world_size()
    dt = getattr(torch, a.dtype)
    es = torch.empty(0, dtype=dt).element_size()
    st = symm.state()
    cap = a.max_mb * 1024 * 1024
    buf = symm.alloc(cap)
    sizes = [1 << k for k in range(10, 31) if (1 << k) <= cap]
    if a.quick:
        sizes = [s_ for s_ in sizes if s_ in (1 << 10, 1 << 16, 1 << 20, 1 << 22, 1 << 25, 1 << 26, 1 << 28, 1 << 30)]
    wire = symm.alloc(cap // 2) if dt == torch.float32 else None
    for nbytes in sizes:
        n = nbytes // es
        quantum = world * (16 // es)
        n = max(quantum, n // quantum * quantum)
        view = buf.view(dt, 0, n)
        view.fill_(1.0)
        ref = torch.ones(n, dtype=dt, device="cuda")
        iters = 50 if nbytes <= (1 << 22) else (10 if nbytes <= (1 << 27) else 4)
        ms_f = timed(lambda: N.allreduce_fused(st, buf, 0, n, dt, view, prescale=1.0 / world, ctas=a.ctas or None), iters, world)
        ms_n = timed(lambda: tdist.all_reduce(ref), iters, world)
        ms_w = None
        if wire is not None and n % (world * 8) == 0:
            local = torch.ones(n, dtype=torch.float32, device="cuda")
            ms_w = timed(lambda: N.allreduce_wire(st, wire, n, torch.bfloat16, local, prescale=1.0 / world,
                                                  ctas=a.ctas or None), iters, world)
            assert torch.allclose(local, torch.ones_like(local), atol=1e-2)
        torch.cuda.synchronize()
        symm.check_status("bench all-reduce")
        roof_ms = 2.0 * (world - 1) / world * nbytes / (LINK_GBS * 1e9) * 1e3
        if rank == 0:
            print(json.dumps({"bytes": nbytes, "n_gpus": world, "dtype": a.dtype, "fused_ms": ms_f, "nccl_ms": ms_n,
                              "fused_busbw_GBs": 2.0 * (world - 1) / world * nbytes / ms_f / 1e6,
                              "nccl_busbw_GBs": 2.0 * (world - 1) / world * nbytes / ms_n / 1e6,
                              "fused_frac_of_roofline_770": roof_ms / ms_f,
                              "fused_frac_of_roofline_900": roof_ms * LINK_GBS / NOMINAL_GBS / ms_f,
                              "wire16_ms": ms_w,
                              "wire16_busbw_GBs_fp32_equiv": None if ms_w is None else
                              2.0 * (world - 1) / world * nbytes / ms_w / 1e6,
                              "speedup_vs_nccl": ms_n / ms_f, "ctas": a.ctas,
                              "nccl_nvls": os.environ.get("NCCL_NVLS_ENABLE", "nccl default")}), flush=True)
    # correctness of the last case: all ones averaged stay ones
    assert torch.allclose(view.float(), torch.ones_like(view.float()), atol=1e-3)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
