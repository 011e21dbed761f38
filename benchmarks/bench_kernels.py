"""Kernel sweep (BASELINE config 5): bf16 matmul M=N=K in {1k..16k}, RMSNorm / softmax over
8192 rows x {1k, 4k, 16k}, fused AdamW, attention.  CUDA-event timing, warm-up, L2 flushed between
timed iterations by writing a 256 MB buffer.  Prints one JSON line per case with the achieved
fraction of the measured peaks (MEASURED_PEAKS.json next to the repo root, else the fallback).

    python benchmarks/bench_kernels.py [--what gemm,norm,addnorm,softmax,adamw,attn] [--quick]
"""
import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import genesis_b200  # noqa: E402,F401
from genesis_b200.ops import dispatch as K  # noqa: E402
from genesis_b200.ops import native as N  # noqa: E402


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["hbm_gbs"], d["bf16_tflops"], "measured"
    return 6650.0, 1590.0, "fallback"


_flush = None


def flush_l2():
    global _flush
    if _flush is None:
        _flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    _flush.fill_(1)


ITERS = 20
_nvml = None


def sm_mhz():
    """Current SM clock (read-only NVML query), or None without NVML."""
    global _nvml
    try:
        import pynvml
        if _nvml is None:
            pynvml.nvmlInit()
            _nvml = pynvml.nvmlDeviceGetHandleByIndex(torch.cuda.current_device())
        return pynvml.nvmlDeviceGetClockInfo(_nvml, pynvml.NVML_CLOCK_SM)
    except Exception:
        return None


last_clock = None


def timeit(fn, iters=None, warmup=3):
    """Median of `iters` CUDA-event timings (L2 flushed before each) after dropping samples outside 1.5 IQR of the
    quartiles; the SM clock sampled right after the last launch is left in `last_clock`."""
    global last_clock
    iters = iters or ITERS
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts, clk = [], []
    for _ in range(iters):
        flush_l2()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        c = sm_mhz()                      # the kernel is still running or has just ended
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b))
        if c:
            clk.append(c)
    ts.sort()
    if len(ts) >= 8:
        q1, q3 = ts[len(ts) // 4], ts[(3 * len(ts)) // 4]
        lo, hi = q1 - 1.5 * (q3 - q1), q3 + 1.5 * (q3 - q1)
        ts = [t for t in ts if lo <= t <= hi] or ts
    clk.sort()
    last_clock = clk[len(clk) // 2] if clk else None
    return ts[len(ts) // 2]


def emit(rec):
    rec["sm_mhz"] = last_clock
    rec.setdefault("repeats", ITERS)
    print(json.dumps(rec), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--what", default="gemm,norm,softmax,adamw")
    ap.add_argument("--quick", action="store_true")
    ap.add_argument("--torch", action="store_true", help="also time the torch/cuBLAS op for comparison")
    ap.add_argument("--attn-shape", default=None, help="B,S,Hq,Hkv,D of a single attention case")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--gemm-shape", default=None, help="M,N,K of a single linear-forward case (y = x @ w^T)")
    a = ap.parse_args()
    global ITERS
    ITERS = a.iters
    hbm, tf, src = peaks()
    what = a.what.split(",")
    dev = "cuda"
    if a.gemm_shape:
        m, nn, k = [int(v) for v in a.gemm_shape.split(",")]
        X = torch.randn(m, k, device=dev, dtype=torch.bfloat16)
        W = torch.randn(nn, k, device=dev, dtype=torch.bfloat16)
        ms = timeit(lambda: K.linear(X, W))
        rec = {"kernel": "linear_fwd", "M": m, "N": nn, "K": k, "ms": ms, "tflops": 2 * m * nn * k / ms / 1e9,
               "frac_of_" + src: 2 * m * nn * k / ms / 1e9 / tf}
        if a.torch:
            rec["torch_ms"] = timeit(lambda: torch.matmul(X, W.t()))
        emit(rec)
        return
    if "gemm" in what:
        # (run first, before the large squares heat the part into its power cap)
        # the shapes of the Qwen2.5-0.5B step (M = 16384 tokens)
        for (m, nn, k, tag) in [(16384, 896, 896, "q/o_proj"), (16384, 4864, 896, "gate/up"), (16384, 896, 4864, "down"),
                                (16384, 151936, 896, "lm_head")]:
            if a.quick and nn > 100000:
                continue
            X = torch.randn(m, k, device=dev, dtype=torch.bfloat16)
            W = torch.randn(nn, k, device=dev, dtype=torch.bfloat16)
            G = torch.randn(m, nn, device=dev, dtype=torch.bfloat16)
            for name, fn in [("fwd", lambda: K.linear(X, W)), ("dgrad", lambda: K.linear_dgrad(G, W)),
                             ("wgrad", lambda: K.linear_wgrad(G, X, out_dtype=torch.float32))]:
                ms = timeit(fn)
                rec = {"kernel": f"linear_{name}", "shape": tag, "M": m, "N": nn, "K": k, "ms": ms,
                       "tflops": 2 * m * nn * k / ms / 1e9, "frac_of_" + src: 2 * m * nn * k / ms / 1e9 / tf}
                if a.torch:
                    tfn = {"fwd": lambda: torch.matmul(X, W.t()), "dgrad": lambda: torch.matmul(G, W),
                           "wgrad": lambda: torch.matmul(G.t(), X)}[name]
                    rec["torch_ms"] = timeit(tfn)
                emit(rec)
            del X, W, G
        sizes = [1024, 2048, 4096, 8192] + ([] if a.quick else [16384])
        for n in sizes:
            A = torch.randn(n, n, device=dev, dtype=torch.bfloat16)
            B = torch.randn(n, n, device=dev, dtype=torch.bfloat16)
            ms = timeit(lambda: N.gemm(A, B))
            rec = {"kernel": "gemm_bf16_tn", "M": n, "N": n, "K": n, "ms": ms, "tflops": 2 * n ** 3 / ms / 1e9,
                   "frac_of_" + src: 2 * n ** 3 / ms / 1e9 / tf}
            if a.torch:
                mt = timeit(lambda: torch.matmul(A, B.t()))
                rec["torch_ms"] = mt
            emit(rec)
    if "norm" in what or "softmax" in what:
        for cols in [1024, 4096, 16384]:
            x = torch.randn(8192, cols, device=dev, dtype=torch.bfloat16)
            w = torch.ones(cols, device=dev)
            if "norm" in what:
                ms = timeit(lambda: K.rmsnorm_fwd(x, w, 1e-6))
                gbs = 2 * x.numel() * 2 / ms / 1e6
                emit({"kernel": "rmsnorm_fwd", "rows": 8192, "cols": cols, "ms": ms, "GBs": gbs,
                                  "frac_of_" + src: gbs / hbm})
            if "softmax" in what:
                ms = timeit(lambda: K.softmax_fwd(x, -1))
                gbs = 2 * x.numel() * 2 / ms / 1e6
                emit({"kernel": "softmax_fwd", "rows": 8192, "cols": cols, "ms": ms, "GBs": gbs,
                                  "frac_of_" + src: gbs / hbm})
                x32 = x.float()                      # the reference's softmax computes in float32: same shapes, twice the bytes
                ms = timeit(lambda: K.softmax_fwd(x32, -1))
                gbs = 2 * x32.numel() * 4 / ms / 1e6
                emit({"kernel": "softmax_fwd_fp32", "rows": 8192, "cols": cols, "ms": ms, "GBs": gbs,
                      "frac_of_" + src: gbs / hbm})
                del x32
    if "addnorm" in what:
        # residual addition + RMSNorm at the residual-stream shape of the 0.5B model (16384 tokens x 896)
        rows, cols = 16384, 896
        x = torch.randn(rows, cols, device=dev, dtype=torch.bfloat16)
        r = torch.randn(rows, cols, device=dev, dtype=torch.bfloat16)
        w = torch.ones(cols, device=dev)
        s_, y_, rstd = K.add_rmsnorm_fwd(x, r, w, 1e-6)
        unit = rows * cols * 2
        ms = timeit(lambda: K.add_rmsnorm_fwd(x, r, w, 1e-6))
        emit({"kernel": "add_rmsnorm_fwd", "rows": rows, "cols": cols, "ms": ms, "GBs": 4 * unit / ms / 1e6,
                          "frac_of_" + src: 4 * unit / ms / 1e6 / hbm})
        ms = timeit(lambda: K.add_rmsnorm_bwd(y_, r, s_, w, rstd))
        emit({"kernel": "add_rmsnorm_bwd", "rows": rows, "cols": cols, "ms": ms, "GBs": 4 * unit / ms / 1e6,
                          "frac_of_" + src: 4 * unit / ms / 1e6 / hbm})
    if "adamw" in what:
        n = 250_000_000 if a.quick else 1_000_000_000
        p = torch.zeros(n, device=dev)
        g = torch.ones(n, device=dev)
        m, v = torch.zeros(n, device=dev), torch.zeros(n, device=dev)
        ms = timeit(lambda: K.adamw_step([p], [g], [m], [v], 1e-3, 0.9, 0.999, 1e-8, 0.01, 1), iters=5)
        gbs = n * 28 / ms / 1e6
        emit({"kernel": "adamw_multi_tensor", "params": n, "ms": ms, "GBs": gbs, "frac_of_" + src: gbs / hbm, "repeats": 5})
    if "attn" in what:
        cases = [(8, S, 16, 4, 128) for S in [1024, 4096] + ([] if a.quick else [16384])]
        if a.attn_shape:
            cases = [tuple(int(x) for x in a.attn_shape.split(","))]
        for (B, S, Hq, Hkv, D) in cases:
            q = torch.randn(B, S, Hq, D, device=dev, dtype=torch.bfloat16)
            k = torch.randn(B, S, Hkv, D, device=dev, dtype=torch.bfloat16)
            v = torch.randn(B, S, Hkv, D, device=dev, dtype=torch.bfloat16)
            r = N.attention_fwd(q, k, v, True, D ** -0.5)
            if r is NotImplemented:
                print(json.dumps({"kernel": "attention_fwd", "S": S, "status": "not implemented"}))
                continue
            ms = timeit(lambda: N.attention_fwd(q, k, v, True, D ** -0.5))
            fl = 4 * B * Hq * S * S * D / 2
            rec = {"kernel": "attention_fwd", "B": B, "S": S, "Hq": Hq, "Hkv": Hkv, "D": D, "ms": ms,
                   "tflops": fl / ms / 1e9}
            o, lse = r
            do = torch.randn_like(o)
            rb = N.attention_bwd(do, q, k, v, o, lse, True, D ** -0.5)
            if rb is not NotImplemented:
                msb = timeit(lambda: N.attention_bwd(do, q, k, v, o, lse, True, D ** -0.5), iters=a.iters,
                             warmup=min(3, a.iters))
                rec.update({"bwd_ms": msb, "bwd_tflops": 2.5 * fl / msb / 1e9})
            emit(rec)
    N.check_status()


if __name__ == "__main__":
    main()
