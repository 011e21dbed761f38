"""Small, self-terminating workloads of single kernel families, sized for profiler captures: inputs larger than the
126 MB L2 where DRAM figures matter, a few hundred MB on the device at most, three launches each.

    python benchmarks/ncu_case.py <case>
    ncu --set full --clock-control none -k regex:<kernel> -c 2 -o prof python benchmarks/ncu_case.py <case>

Cases (kernel to pass to -k): gemm_pair, gemm_swiglu, gemm_swiglu_bwd (gemm2_kernel), gemm (gemm_kernel),
grouped_gemm (gemm_kernel), attn128_fwd (attn_fwd_kernel), attn128_bwd (attn_bwd_dq_kernel / attn_bwd_dkdv_kernel),
attn64_fwd, attn64_bwd, ce (ce_fwd_kernel / ce_bwd_kernel), softmax (row_stream_kernel / softmax_bwd), rmsnorm (row_stream_kernel / rmsnorm_bwd_kernel),
addnorm, adam (adam_multi_kernel), swiglu_bwd (swiglu_bwd2d_kernel), rope (rope_vec_kernel),
reduce_cols (reduce_mid), sort (sort_rows), index (index_get_kernel / index_put_kernel), cat (cat_kernel).
"""
import sys
import os

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import genesis_b200 as genesis  # noqa: E402
from genesis_b200.ops import dispatch as K  # noqa: E402
from genesis_b200.ops import native as N  # noqa: E402

DEV = "cuda"
BF = torch.bfloat16


def rnd(*shape, dt=BF, scale=1.0):
    return (torch.randn(*shape, device=DEV) * scale).to(dt)


def gemm_pair():
    a, b = rnd(8192, 4096), rnd(4096, 4096)
    N.pair_mode = "1"
    return lambda: N.gemm(a, b)


def gemm_swiglu():
    x, w = rnd(16384, 896), rnd(9728, 896, scale=0.05)
    return lambda: N.linear_swiglu(x, w)


def gemm_swiglu_bwd():
    gy, wd_t, gu = rnd(16384, 896), rnd(4864, 896, scale=0.05), rnd(16384, 9728)
    return lambda: N.dgrad_swiglu_bwd(gy, wd_t, gu)


def gemm():
    a, b = rnd(8192, 4096), rnd(4096, 4096)
    N.pair_mode = "0"
    return lambda: N.gemm(a, b)


def grouped_gemm():
    E, H, I, rows = 16, 2048, 768, 4096
    x = rnd(E * rows, H)
    w = rnd(E, 2 * I, H, scale=0.05)
    off = (torch.arange(E + 1, device=DEV) * rows).to(torch.int32)
    return lambda: K.grouped_linear(x, w, off)


def _attn(B, S, Hq, Hkv, D, bwd):
    q, k, v = rnd(B, S, Hq, D), rnd(B, S, Hkv, D), rnd(B, S, Hkv, D)
    scale = D ** -0.5
    if not bwd:
        return lambda: K.attention_fwd(q, k, v, True, scale)
    o, lse = K.attention_fwd(q, k, v, True, scale)
    do = rnd(B, S, Hq, D)
    return lambda: K.attention_bwd(do, q, k, v, o, lse, True, scale)


def ce():
    logits = rnd(4096, 151936)
    tgt = torch.randint(0, 151936, (4096,), device=DEV)

    def f():
        loss_rows, lse = K.cross_entropy_fwd(logits, tgt, -100)
        K.cross_entropy_bwd(logits, tgt, lse, torch.ones(4096, device=DEV) / 4096, -100)
    return f


def softmax():
    x = rnd(8192, 16384)

    def f():
        y = K.softmax_fwd(x, -1)
        K.softmax_bwd(y, y, -1)
    return f


def rmsnorm():
    x, w, g = rnd(8192, 16384), torch.ones(16384, device=DEV), rnd(8192, 16384)

    def f():
        y, rstd = K.rmsnorm_fwd(x, w, 1e-6)
        K.rmsnorm_bwd(g, x, w, rstd)
    return f


def addnorm():
    x, r, w, g = rnd(65536, 896), rnd(65536, 896), torch.ones(896, device=DEV), rnd(65536, 896)

    def f():
        s, y, rstd = K.add_rmsnorm_fwd(x, r, w, 1e-6)
        K.add_rmsnorm_bwd(g, g, s, w, rstd)
    return f


def adam():
    ps = [torch.randn(64 * 1024 * 1024 // 8, device=DEV) for _ in range(8)]
    gs = [torch.randn_like(p) for p in ps]
    ms, vs = [torch.zeros_like(p) for p in ps], [torch.zeros_like(p) for p in ps]
    return lambda: K.adamw_step(ps, gs, ms, vs, 1e-3, 0.9, 0.999, 1e-8, 0.01, 1)


def swiglu_bwd():
    gu, dy = rnd(16384, 9728), rnd(16384, 4864)
    return lambda: K.swiglu_fused_bwd(dy, gu)


def rope():
    from genesis_b200.models.transformers.components import RotaryEmbedding
    rot = RotaryEmbedding(64, max_position_embeddings=2048, base=1e6)
    rot._build(2048)
    x = rnd(16, 2048, 14, 64)
    cos, sin = rot.cos_cached._t.to(DEV), rot.sin_cached._t.to(DEV)
    return lambda: K.rope_fwd(x, cos, sin, None, False)


def reduce_cols():
    x = rnd(65536, 1152)
    return lambda: K.reduce("sum", x, (0,), False)


def sort():
    x = rnd(8192, 4096, dt=torch.float32)
    return lambda: K.sort(x, -1, False)


def index():
    a = rnd(65536, 1024)
    i = torch.randint(0, 65536, (65536,), device=DEV)
    g = rnd(65536, 1024)

    def f():
        K.getitem(a, (i,))
        K.getitem_backward((65536, 1024), (i,), g)
    return f


def cat():
    xs = [rnd(16384, 1024) for _ in range(4)]
    return lambda: K.cat(xs, 1)


CASES = {
    "gemm_pair": gemm_pair, "gemm_swiglu": gemm_swiglu, "gemm_swiglu_bwd": gemm_swiglu_bwd, "gemm": gemm, "grouped_gemm": grouped_gemm,
    "attn128_fwd": lambda: _attn(4, 4096, 16, 4, 128, False), "attn128_bwd": lambda: _attn(4, 4096, 16, 4, 128, True),
    "attn64_fwd": lambda: _attn(8, 2048, 14, 2, 64, False), "attn64_bwd": lambda: _attn(8, 2048, 14, 2, 64, True),
    "ce": ce, "softmax": softmax, "rmsnorm": rmsnorm, "addnorm": addnorm, "adam": adam, "swiglu_bwd": swiglu_bwd,
    "rope": rope, "reduce_cols": reduce_cols, "sort": sort, "index": index, "cat": cat,
}


def main():
    name = sys.argv[1]
    fn = CASES[name]()
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    N.check_status()
    print(f"{name}: ok, fallbacks {K.fallback_counts()}")


if __name__ == "__main__":
    main()
