"""tcgen05 flash attention (forward, dQ, dK/dV) against an fp32 softmax(QK^T)V reference."""
import pytest
import torch

import genesis_b200  # noqa: F401
from genesis_b200.ops import dispatch as K
from genesis_b200.ops import native as N

pytestmark = pytest.mark.gpu
DEV = "cuda"


def rnd(*shape, dt, seed=0):
    g = torch.Generator().manual_seed(seed + sum(shape))
    return torch.randn(*shape, generator=g).to(dt)


CASES = [
    # B, S, Sk, Hq, Hkv, D, causal
    (1, 128, 128, 1, 1, 64, True), (2, 256, 256, 4, 2, 64, True), (1, 100, 100, 2, 1, 64, True),
    (2, 384, 384, 6, 2, 128, True), (1, 130, 130, 3, 3, 128, False), (1, 512, 512, 14, 2, 64, True),
    (1, 64, 320, 2, 1, 64, True), (1, 200, 200, 2, 2, 128, True), (1, 1024, 1024, 2, 1, 128, True),
    (1, 257, 257, 2, 1, 64, False),
]


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("case", CASES)
def test_attention_fwd_bwd(dt, case):
    B, S, Sk, Hq, Hkv, D, causal = case
    q, k, v = rnd(B, S, Hq, D, dt=dt), rnd(B, Sk, Hkv, D, dt=dt, seed=1), rnd(B, Sk, Hkv, D, dt=dt, seed=2)
    do = rnd(B, S, Hq, D, dt=dt, seed=3)
    scale = D ** -0.5
    o_ref, lse_ref = K.attention_fwd(q.float(), k.float(), v.float(), causal, scale)
    r = N.attention_fwd(q.to(DEV), k.to(DEV), v.to(DEV), causal, scale)
    assert r is not NotImplemented
    o, lse = r
    N.check_status()
    tol = 2e-2 if dt == torch.bfloat16 else 4e-3
    torch.testing.assert_close(o.float().cpu(), o_ref, atol=tol, rtol=tol)
    torch.testing.assert_close(lse.cpu(), lse_ref, atol=2e-3, rtol=2e-3)
    dq_ref, dk_ref, dv_ref = K.attention_bwd(do.float(), q.float(), k.float(), v.float(), o_ref, lse_ref, causal, scale)
    rb = N.attention_bwd(do.to(DEV), q.to(DEV), k.to(DEV), v.to(DEV), o, lse, causal, scale)
    assert rb is not NotImplemented
    N.check_status()
    dq, dk, dv = rb
    g = Hq // Hkv
    btol = tol * 4 * max(1.0, g ** 0.5)
    torch.testing.assert_close(dq.float().cpu(), dq_ref, atol=btol, rtol=5e-2)
    torch.testing.assert_close(dk.float().cpu(), dk_ref, atol=btol, rtol=5e-2)
    torch.testing.assert_close(dv.float().cpu(), dv_ref, atol=btol, rtol=5e-2)


def test_attention_through_autograd():
    import genesis_b200 as genesis
    import genesis_b200.nn.functional as F
    B, S, Hq, Hkv, D = 2, 256, 4, 2, 64
    qa, ka, va = rnd(B, S, Hq, D, dt=torch.float32), rnd(B, S, Hkv, D, dt=torch.float32, seed=1), \
        rnd(B, S, Hkv, D, dt=torch.float32, seed=2)
    outs = []
    for dev in ("cpu", "cuda"):
        q, k, v = (genesis.Tensor(t.to(dev), requires_grad=True) for t in (qa, ka, va))
        if dev == "cuda":
            with genesis.amp.autocast(dtype=genesis.bfloat16):
                o = F.flash_attention(q, k, v, causal=True)
        else:
            o = F.flash_attention(q, k, v, causal=True)
        (o.float() * o.float()).sum().backward()
        outs.append((o._t.float().cpu(), q.grad._t.float().cpu(), k.grad._t.float().cpu(), v.grad._t.float().cpu()))
    for a, b in zip(*outs):
        torch.testing.assert_close(b, a, atol=6e-2, rtol=6e-2)
