"""Kernels that promise a fixed summation order give bit-identical results when run twice (two-stage reductions, norms'
weight gradients, whole-tile GEMMs, attention forward, attention backward without head groups).  The paths that add
partial results in memory (stream-K / split-K GEMM, dK/dV of grouped-query attention) are excluded by design."""
import pytest
import torch

from genesis_b200.ops import dispatch as K
from genesis_b200.ops import native as N

pytestmark = pytest.mark.gpu


def _twice(fn):
    a = fn()
    b = fn()
    a = a if isinstance(a, (tuple, list)) else (a,)
    b = b if isinstance(b, (tuple, list)) else (b,)
    torch.cuda.synchronize()
    for x, y in zip(a, b):
        assert torch.equal(x, y)


def test_reductions_and_norm_weight_gradients_are_reproducible():
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn(4096, 1536, device="cuda", generator=g).bfloat16()
    gy = torch.randn(4096, 1536, device="cuda", generator=g).bfloat16()
    w = torch.randn(1536, device="cuda", generator=g)
    _twice(lambda: K.reduce("sum", x.float(), None, False))
    _twice(lambda: K.reduce("sum", x, (0,), False))
    _twice(lambda: K.reduce("sum", x, (1,), False))
    y, rstd = K.rmsnorm_fwd(x, w, 1e-6)
    _twice(lambda: K.rmsnorm_bwd(gy, x, w, rstd))
    yl, mean, rs = K.layernorm_fwd(x, w, w, 1e-5)
    _twice(lambda: K.layernorm_bwd(gy, x, w, mean, rs))
    _twice(lambda: K.bias_grad(gy, torch.float32))


def test_whole_tile_gemm_and_cross_entropy_are_reproducible():
    g = torch.Generator(device="cuda").manual_seed(1)
    a = torch.randn(2048, 1024, device="cuda", generator=g).bfloat16()
    b = torch.randn(3072, 1024, device="cuda", generator=g).bfloat16()
    _twice(lambda: K.linear(a, b))
    _twice(lambda: K.linear_dgrad(K.linear(a, b), b))
    logits = torch.randn(512, 151936, device="cuda", generator=g).bfloat16()
    tgt = torch.randint(0, 151936, (512,), device="cuda", generator=g)
    _twice(lambda: K.cross_entropy_fwd(logits, tgt, -100))


@pytest.mark.parametrize("Hq,Hkv,D", [(4, 4, 64), (4, 4, 128)])
def test_attention_is_reproducible_without_head_groups(Hq, Hkv, D):
    g = torch.Generator(device="cuda").manual_seed(2)
    q = torch.randn(2, 512, Hq, D, device="cuda", generator=g).bfloat16()
    k = torch.randn(2, 512, Hkv, D, device="cuda", generator=g).bfloat16()
    v = torch.randn(2, 512, Hkv, D, device="cuda", generator=g).bfloat16()
    _twice(lambda: N.attention_fwd(q, k, v, True, D ** -0.5))
    o, lse = N.attention_fwd(q, k, v, True, D ** -0.5)
    do = torch.randn_like(o)
    _twice(lambda: N.attention_bwd(do, q, k, v, o, lse, True, D ** -0.5))
