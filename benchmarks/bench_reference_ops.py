"""Times single ops of the UNMODIFIED reference package (installed under baseline/_ref) through its public API, at the
shapes of the kernel sweep: the "ref" column of the per-kernel tables.

    python benchmarks/bench_reference_ops.py --family matmul|rmsnorm|softmax|attention [--iters 5]

One op family per process and few iterations.  Only shapes whose tensors stay far below 2**31 elements are run: the
reference's elementwise kernels index with 32-bit offsets, which is what faulted its full training step (the
[tokens, vocab] loss temporaries); nothing here comes near that.  S = 16384 attention is left out (outside the list
its fused kernel accepts; its fallback would materialise a score matrix of 3.4e10 elements).  A case that raises is
reported with its message and the sweep goes on.  CUDA-event timing, L2 flushed between iterations, one JSON line
per case.  `genesis` here is the reference, not this framework: its install directory leads `sys.path`.
"""
import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--family", required=True, choices=["matmul", "rmsnorm", "softmax", "attention"])
    ap.add_argument("--iters", type=int, default=5)
    a = ap.parse_args()
    if not os.path.isdir(os.path.join(REF, "genesis")):
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref/genesis is not installed"}))
        return
    sys.path.insert(0, REF)
    import numpy as np
    import torch
    import genesis                                   # the reference
    assert os.path.realpath(genesis.__file__).startswith(os.path.realpath(REF)), genesis.__file__
    import genesis.nn.functional as F
    dev = genesis.device("cuda")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")

    def timed(fn):
        for _ in range(2):
            fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(a.iters):
            flush.fill_(1)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        ts.sort()
        return ts[len(ts) // 2]

    def rand(*shape, dtype=genesis.float32):
        t = genesis.tensor(np.random.RandomState(0).randn(*shape).astype(np.float32), device=dev)
        return t if dtype == genesis.float32 else t.to_dtype(dtype)

    def report(rec, fn):
        try:
            rec["ms"] = timed(fn)
        except Exception as e:                       # recorded verbatim, the sweep goes on
            rec["error"] = f"{type(e).__name__}: {str(e)[:300]}"
        rec["impl"] = "reference"
        print(json.dumps(rec), flush=True)

    if a.family == "matmul":
        for n in (1024, 2048, 4096, 8192, 16384):
            A, B = rand(n, n, dtype=genesis.bfloat16), rand(n, n, dtype=genesis.bfloat16)
            rec = {"op": "matmul bf16", "M": n, "N": n, "K": n, "dtype": str(A.dtype)}
            report(rec, lambda: genesis.matmul(A, B))
            if "ms" in rec:
                print(json.dumps({"op": "matmul bf16", "n": n, "tflops": 2.0 * n ** 3 / rec["ms"] / 1e9}), flush=True)
            del A, B
    elif a.family == "rmsnorm":
        from genesis.nn.triton_ops import fused_rmsnorm
        for cols in (1024, 4096, 16384):
            x = rand(8192, cols, dtype=genesis.bfloat16)
            w = genesis.tensor(np.ones(cols, np.float32), device=dev)
            rec = {"op": "rmsnorm fwd", "rows": 8192, "cols": cols, "dtype": str(x.dtype)}
            report(rec, lambda: fused_rmsnorm(x, w, 1e-6))
            del x
    elif a.family == "softmax":
        for cols in (1024, 4096, 16384):
            x = rand(8192, cols)                     # the reference's softmax computes in float32
            rec = {"op": "softmax fwd", "rows": 8192, "cols": cols, "dtype": str(x.dtype)}
            report(rec, lambda: F.softmax(x, dim=-1))
            del x
    else:
        for S in (1024, 4096):
            # Hq = 16, Hkv = 4 in the sweep; the reference's fused kernel needs Hq == Hkv, so K and V arrive
            # replicated to 16 heads (the copy is not timed)
            q = rand(8, 16, S, 128, dtype=genesis.float16)
            k = rand(8, 16, S, 128, dtype=genesis.float16)
            v = rand(8, 16, S, 128, dtype=genesis.float16)
            rec = {"op": "causal attention fwd", "B": 8, "H": 16, "S": S, "D": 128, "dtype": str(q.dtype)}
            report(rec, lambda: F.scaled_dot_product_attention(q, k, v))
            if "ms" in rec:
                fl = 4.0 * 8 * 16 * S * S * 128 / 2
                print(json.dumps({"op": "attention", "S": S, "tflops": fl / rec["ms"] / 1e9}), flush=True)
            del q, k, v


if __name__ == "__main__":
    main()
