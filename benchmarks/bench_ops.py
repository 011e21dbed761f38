"""Operator sweep against torch on the same GPU: a registry of ops x shapes, CUDA-event timing with warm-up, IQR
outlier filtering and medians, GB/s (algorithmic bytes) or TFLOP/s per case, a markdown report.

    python benchmarks/bench_ops.py [--category elementwise,reduction,norm,matmul,index] [--dtype bf16] [--report out.md]

Each case times `genesis_b200` (the framework's own kernels through its public Tensor API, so Python dispatch is
included: `--timing real`) or only the raw kernel entry point (`--timing pure`).  Between iterations a 256 MB
buffer is overwritten so inputs never sit in the 126 MB L2.
Reference counterpart: benchmark/bench_ops.py (registry, IQR filter, markdown report).
"""
import argparse
import json
import os
import statistics
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def iqr_median(samples):
    """Median after dropping samples outside [q1 - 1.5 iqr, q3 + 1.5 iqr]."""
    s = sorted(samples)
    if len(s) < 4:
        return statistics.median(s)
    q1, q3 = s[len(s) // 4], s[(3 * len(s)) // 4]
    lo, hi = q1 - 1.5 * (q3 - q1), q3 + 1.5 * (q3 - q1)
    kept = [v for v in s if lo <= v <= hi] or s
    return statistics.median(kept)


def time_ms(torch, fn, flush, iters=20, warmup=5):
    for _ in range(warmup):
        fn()
    out = []
    for _ in range(iters):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        out.append(e0.elapsed_time(e1))
    return iqr_median(out)


def build_cases(torch, genesis, F, K, dt, categories):
    """(category, name, shape text, ours(), theirs(), bytes moved, flops) per case."""
    g = genesis.Tensor
    es = torch.empty(0, dtype=dt).element_size()
    cases = []

    def rnd(*shape, dtype=dt):
        return torch.randn(*shape, device="cuda", dtype=dtype)

    if "elementwise" in categories:
        for n in (256, 2048, 4096, 8192):
            a, b = rnd(n, n), rnd(n, n)
            ga, gb_ = g(a), g(b)
            nb = n * n * es
            cases += [("elementwise", "add", f"{n}x{n}", lambda ga=ga, gb_=gb_: ga + gb_, lambda a=a, b=b: a + b, 3 * nb, 0),
                      ("elementwise", "mul", f"{n}x{n}", lambda ga=ga, gb_=gb_: ga * gb_, lambda a=a, b=b: a * b, 3 * nb, 0),
                      ("elementwise", "exp", f"{n}x{n}", lambda ga=ga: F.exp(ga), lambda a=a: torch.exp(a), 2 * nb, 0),
                      ("elementwise", "silu", f"{n}x{n}", lambda ga=ga: F.silu(ga), lambda a=a: torch.nn.functional.silu(a), 2 * nb, 0),
                      ("elementwise", "add scalar", f"{n}x{n}", lambda ga=ga: ga + 1.5, lambda a=a: a + 1.5, 2 * nb, 0)]
    if "reduction" in categories:
        for n in (1024, 4096, 8192):
            a = rnd(n, n)
            ga = g(a)
            nb = n * n * es
            cases += [("reduction", "sum all", f"{n}x{n}", lambda ga=ga: ga.sum(), lambda a=a: a.sum(), nb, 0),
                      ("reduction", "sum rows (last dim)", f"{n}x{n}", lambda ga=ga: ga.sum(-1), lambda a=a: a.sum(-1), nb, 0),
                      ("reduction", "sum cols (dim 0)", f"{n}x{n}", lambda ga=ga: ga.sum(0), lambda a=a: a.sum(0), nb, 0),
                      ("reduction", "max rows", f"{n}x{n}", lambda ga=ga: ga.max(-1), lambda a=a: a.amax(-1), nb, 0)]
    if "norm" in categories:
        for cols in (1024, 4096, 16384):
            x = rnd(8192, cols)
            w = torch.ones(cols, device="cuda", dtype=dt)
            gx, gw = g(x), g(w)
            nb = 2 * x.numel() * es
            cases += [("norm", "rmsnorm", f"8192x{cols}", lambda gx=gx, gw=gw: F.rms_norm(gx, gw, 1e-6),
                       lambda x=x, w=w: torch.nn.functional.rms_norm(x, (x.shape[-1],), w.to(x.dtype), 1e-6), nb, 0),
                      ("norm", "layernorm", f"8192x{cols}", lambda gx=gx, gw=gw: F.layer_norm(gx, gw, gw, 1e-5),
                       lambda x=x, w=w: torch.nn.functional.layer_norm(x, (x.shape[-1],), w.to(x.dtype), w.to(x.dtype), 1e-5), nb, 0),
                      ("norm", "softmax", f"8192x{cols}", lambda gx=gx: F.softmax(gx, -1),
                       lambda x=x: torch.softmax(x, -1), nb, 0)]
    if "matmul" in categories:
        for n in (1024, 2048, 4096, 8192):
            a, b = rnd(n, n), rnd(n, n)
            ga, gb_ = g(a), g(b)
            cases.append(("matmul", "matmul", f"{n}^3", lambda ga=ga, gb_=gb_: ga @ gb_, lambda a=a, b=b: a @ b, 0, 2 * n ** 3))
        a3, b3 = rnd(32, 1024, 512), rnd(32, 512, 1024)
        cases.append(("matmul", "bmm", "32x1024x512x1024", lambda a3=g(a3), b3=g(b3): a3 @ b3, lambda a3=a3, b3=b3: a3 @ b3,
                      0, 2 * 32 * 1024 * 512 * 1024))
    if "index" in categories:
        table = rnd(151936, 896)
        ids = torch.randint(0, 151936, (16384,), device="cuda")
        gt, gi = g(table), g(ids)
        cases.append(("index", "embedding rows", "16384 of 151936x896", lambda gt=gt, gi=gi: F.embedding(gt, gi),
                      lambda table=table, ids=ids: table[ids], 2 * 16384 * 896 * es, 0))
        x = torch.randn(4096, 4096, device="cuda")
        cases += [("index", "topk 8", "4096x4096 fp32", lambda: K.topk(x, 8, -1, True), lambda: torch.topk(x, 8, -1), x.numel() * 4, 0),
                  ("index", "sort", "4096x4096 fp32", lambda: K.sort(x, -1, False), lambda: torch.sort(x, dim=-1, stable=True), 2 * x.numel() * 4, 0),
                  ("index", "argmax", "4096x4096 fp32", lambda: K.argmax(x, -1), lambda: torch.argmax(x, -1), x.numel() * 4, 0)]
    return cases


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--category", default="elementwise,reduction,norm,matmul,index")
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp16", "fp32"])
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--report", default=None, help="write a markdown table here")
    a = ap.parse_args()
    import torch
    import genesis_b200 as genesis
    import genesis_b200.nn.functional as F
    from genesis_b200.ops import dispatch as K
    from genesis_b200.ops import native
    dt = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}[a.dtype]
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    rows = []
    with genesis.no_grad():
        for cat, name, shape, ours, theirs, nbytes, flops in build_cases(torch, genesis, F, K, dt, a.category.split(",")):
            try:
                mo = time_ms(torch, ours, flush, a.iters)
                mt = time_ms(torch, theirs, flush, a.iters)
            except Exception as e:                                   # keep the sweep going, report the case
                print(json.dumps({"category": cat, "op": name, "shape": shape, "error": str(e)[:200]}), flush=True)
                continue
            rec = {"category": cat, "op": name, "shape": shape, "dtype": a.dtype, "ms": mo, "torch_ms": mt,
                   "speedup_vs_torch": mt / mo}
            if nbytes:
                rec["GBs"] = nbytes / mo / 1e6
            if flops:
                rec["tflops"] = flops / mo / 1e9
            rows.append(rec)
            print(json.dumps(rec), flush=True)
    native.check_status()
    if a.report:
        with open(a.report, "w") as f:
            f.write("| category | op | shape | ms | torch ms | vs torch | GB/s | TFLOP/s |\n|---|---|---|---|---|---|---|---|\n")
            for r in rows:
                f.write(f"| {r['category']} | {r['op']} | {r['shape']} | {r['ms']:.4f} | {r['torch_ms']:.4f} | "
                        f"{r['speedup_vs_torch']:.2f}x | {r.get('GBs', 0):.0f} | {r.get('tflops', 0):.1f} |\n")


if __name__ == "__main__":
    main()
