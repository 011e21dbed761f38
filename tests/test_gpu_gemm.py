"""tcgen05 GEMM against an fp32 torch reference: every operand-layout combination, dtypes,
tile tails, odd (repacked) shapes, bias / accumulate epilogues, batched matmul, linear
forward / dgrad / wgrad."""
import pytest
import torch

import genesis_b200  # noqa: F401
from genesis_b200.ops import dispatch as K
from genesis_b200.ops import native as N

pytestmark = pytest.mark.gpu
DEV = "cuda"


def rnd(*shape, dt=torch.float32, seed=0):
    g = torch.Generator().manual_seed(seed + sum(shape))
    return (torch.randn(*shape, generator=g) * 0.5).to(dt)


def check(got, ref, dt, K_):
    tol = {torch.float32: 5e-3, torch.bfloat16: 2e-2, torch.float16: 4e-3}[dt] * max(1.0, (K_ / 64) ** 0.5)
    torch.testing.assert_close(got.float().cpu(), ref, atol=tol, rtol=2e-2)
    N.check_status()


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("a_mn,b_mn", [(0, 0), (0, 1), (1, 0), (1, 1)])
@pytest.mark.parametrize("M,N_,K_", [(128, 128, 64), (128, 256, 128), (256, 512, 256), (200, 136, 72),
                                      (64, 64, 64), (1024, 896, 896), (8, 8, 8), (384, 4864, 896)])
def test_gemm_layouts(dt, a_mn, b_mn, M, N_, K_):
    a, b = rnd(M, K_, dt=dt), rnd(N_, K_, dt=dt, seed=1)
    ref = a.float() @ b.float().t()
    ac = a.to(DEV).t().contiguous().t() if a_mn else a.to(DEV)
    bc = b.to(DEV).t().contiguous().t() if b_mn else b.to(DEV)
    got = N.gemm(ac, bc)
    assert got is not NotImplemented and got.dtype == dt
    check(got, ref, dt, K_)


@pytest.mark.parametrize("shape", [(3, 4, 5), (5, 4, 3), (16, 16, 32), (72, 73, 74), (74, 73, 72), (1024, 1024, 1024),
                                   (1, 7, 1), (130, 1, 33)])
def test_gemm_odd_shapes(shape):
    m, n, p = shape
    a, b = rnd(m, n), rnd(n, p, seed=1)
    got = K.matmul(a.to(DEV), b.to(DEV))
    check(got, a @ b, torch.float32, n)
    a16, b16 = a.bfloat16(), b.bfloat16()
    got = K.matmul(a16.to(DEV), b16.to(DEV))
    check(got, a16.float() @ b16.float(), torch.bfloat16, n)


def test_gemm_epilogues():
    M, N_, K_ = 300, 264, 200
    a, b, bias = rnd(M, K_, dt=torch.bfloat16), rnd(N_, K_, dt=torch.bfloat16, seed=1), rnd(N_, seed=2)
    ref = a.float() @ b.float().t()
    got = N.gemm(a.to(DEV), b.to(DEV), bias=bias.to(DEV))
    check(got, ref + bias, torch.bfloat16, K_)
    got = N.gemm(a.to(DEV), b.to(DEV), out_dtype=torch.float32)
    assert got.dtype == torch.float32
    check(got, ref, torch.float32, K_)
    acc = rnd(M, N_, seed=3).to(DEV)
    base = acc.clone().cpu()
    N.gemm(a.to(DEV), b.to(DEV), out_dtype=torch.float32, accum=acc)
    check(acc, ref + base, torch.float32, K_)
    got = N.gemm(a.to(DEV), b.to(DEV), alpha=0.25)
    check(got, ref * 0.25, torch.bfloat16, K_)


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("form", ["bmk_bkn", "bmk_kn", "mk_bkn"])
@pytest.mark.parametrize("dims", [(16, 16, 16, 16), (32, 16, 8, 24), (32, 13, 8, 15), (3, 130, 72, 200)])
def test_batched_matmul(dt, form, dims):
    bsz, m, n, p = dims
    a = rnd(bsz, m, n, dt=dt) if form != "mk_bkn" else rnd(m, n, dt=dt)
    b = rnd(bsz, n, p, dt=dt, seed=1) if form != "bmk_kn" else rnd(n, p, dt=dt, seed=1)
    got = K.matmul(a.to(DEV), b.to(DEV))
    check(got, a.float() @ b.float(), dt, n)


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16, torch.float32])
def test_linear_fwd_bwd(dt):
    x, w, b = rnd(4, 50, 896, dt=dt), rnd(136, 896, dt=dt, seed=1), rnd(136, seed=2)
    gy = rnd(4, 50, 136, dt=dt, seed=3)
    y = K.linear(x.to(DEV), w.to(DEV), b.to(DEV))
    check(y, torch.nn.functional.linear(x.float(), w.float(), b), dt, 896)
    dx = K.linear_dgrad(gy.to(DEV), w.to(DEV))
    check(dx, gy.float() @ w.float(), dt, 136)
    dw = K.linear_wgrad(gy.to(DEV), x.to(DEV), out_dtype=torch.float32)
    assert dw.dtype == torch.float32
    check(dw, gy.float().reshape(-1, 136).t() @ x.float().reshape(-1, 896), torch.float32 if dt == torch.float32
          else dt, 200)
    acc = torch.ones(136, 896, device=DEV)
    K.linear_wgrad(gy.to(DEV), x.to(DEV), out_dtype=torch.float32, accum=acc)
    check(acc, 1.0 + gy.float().reshape(-1, 136).t() @ x.float().reshape(-1, 896), torch.float32
          if dt == torch.float32 else dt, 200)


def test_large_gemm_many_tiles():
    # more tiles than SMs: exercises the persistent loop, both accumulators and the smem ring wrap-around
    M, N_, K_ = 2048, 4096, 1024
    a, b = rnd(M, K_, dt=torch.bfloat16), rnd(N_, K_, dt=torch.bfloat16, seed=1)
    got = N.gemm(a.to(DEV), b.to(DEV))
    check(got, a.float() @ b.float().t(), torch.bfloat16, K_)


@pytest.mark.parametrize("M,N_,K_", [(896, 896, 8192), (128, 896, 16384), (4864, 896, 4096), (300, 520, 6000)])
def test_weight_gradient_shapes_split_k(M, N_, K_):
    # small outputs with a long contraction: the planner spreads the k range of the tiles over all SMs
    # (stream-K) and the partial tiles are added into the output by the epilogue
    gy, x = rnd(K_, M, dt=torch.bfloat16), rnd(K_, N_, dt=torch.bfloat16, seed=1)
    ref = gy.float().t() @ x.float()
    got = K.linear_wgrad(gy.to(DEV), x.to(DEV), out_dtype=torch.float32)
    check(got, ref, torch.bfloat16, K_ / 16)
    acc = torch.full((M, N_), 2.0, device=DEV)
    K.linear_wgrad(gy.to(DEV), x.to(DEV), out_dtype=torch.float32, accum=acc)
    check(acc, ref + 2.0, torch.bfloat16, K_ / 16)


@pytest.mark.parametrize("plan", [(256, -1), (128, -1), (256, 3), (128, 1), (256, 1)])
@pytest.mark.parametrize("M,N_,K_", [(640, 1000, 2500), (4864, 896, 2048)])
def test_forced_tile_and_split_plans_agree(plan, M, N_, K_):
    from genesis_b200.ops import native
    gy, x = rnd(K_, M, dt=torch.bfloat16), rnd(K_, N_, dt=torch.bfloat16, seed=3)
    ref = gy.float().t() @ x.float()
    native.plan_override = plan
    try:
        got = K.linear_wgrad(gy.to(DEV), x.to(DEV), out_dtype=torch.float32)
        acc = torch.full((M, N_), -1.5, device=DEV)
        K.linear_wgrad(gy.to(DEV), x.to(DEV), out_dtype=torch.float32, accum=acc)
    finally:
        native.plan_override = None
    check(got, ref, torch.bfloat16, K_ / 16)
    check(acc, ref - 1.5, torch.bfloat16, K_ / 16)


# ---------------------------------------------------------------------------------------------------------
# CTA-pair kernel (csrc/gemm2_sm100.cu): tcgen05.mma.cta_group::2 on clusters of two CTAs
# ---------------------------------------------------------------------------------------------------------
def _pair(a, b_t, out_dtype=None, bias=None, accum=None, bn=256):
    M, K_ = a.shape
    a2, a_mn, lda = N._operand(a, True)
    b2, b_mn, ldb = N._operand(b_t, True)
    out = accum if accum is not None else torch.empty(M, b_t.shape[0], dtype=out_dtype or a.dtype, device=a.device)
    assert N.gemm_pair(a2, a_mn, lda, b2, b_mn, ldb, M, b_t.shape[0], K_, out, bias, accum is not None, 1.0, bn)
    return out


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("M,N_,K_,bn", [(256, 256, 64, 256), (512, 512, 896, 256), (384, 320, 200, 256),
                                         (1024, 896, 896, 128), (1024, 1152, 896, 192), (300, 136, 72, 128),
                                         (2048, 4864, 896, 256), (130, 264, 520, 192)])
def test_pair_gemm_shapes(dt, M, N_, K_, bn):
    a, b = rnd(M, K_, dt=dt), rnd(N_, K_, dt=dt, seed=1)
    got = _pair(a.to(DEV), b.to(DEV), bn=bn)
    check(got, a.float() @ b.float().t(), dt, K_)


@pytest.mark.parametrize("a_mn,b_mn", [(0, 1), (1, 0), (1, 1)])
def test_pair_gemm_layouts_and_epilogues(a_mn, b_mn):
    M, N_, K_ = 768, 640, 448
    a, b, bias = rnd(M, K_, dt=torch.float16), rnd(N_, K_, dt=torch.float16, seed=1), rnd(N_, seed=2)
    ref = a.float() @ b.float().t()
    ac = a.to(DEV).t().contiguous().t() if a_mn else a.to(DEV)
    bc = b.to(DEV).t().contiguous().t() if b_mn else b.to(DEV)
    check(_pair(ac, bc, bn=128 if b_mn else 192), ref, torch.float16, K_)
    check(_pair(ac, bc, out_dtype=torch.float32, bias=bias.to(DEV)), ref + bias, torch.float16, K_)
    acc = torch.ones(M, N_, device=DEV)
    check(_pair(ac, bc, accum=acc), ref + 1.0, torch.float16, K_)


@pytest.mark.parametrize("M,I,K_", [(256, 128, 64), (512, 256, 896), (1000, 384, 200), (2048, 4864, 896)])
def test_pair_gemm_swiglu_epilogue(M, I, K_):
    x = rnd(M, K_, dt=torch.bfloat16)
    w = (rnd(2 * I, K_, seed=1) * 0.2).bfloat16()
    gu_ref = x.float() @ w.float().t()
    h_ref = torch.nn.functional.silu(gu_ref[:, :I]) * gu_ref[:, I:]
    gu, h = N.linear_swiglu(x.to(DEV), w.to(DEV))
    check(gu, gu_ref, torch.bfloat16, K_)
    check(h, h_ref, torch.bfloat16, K_)
    _, h2 = N.linear_swiglu(x.to(DEV), w.to(DEV), want_gu=False)
    assert torch.equal(h, h2)


def test_linear_swiglu_function_matches_the_unfused_layers():
    import genesis_b200 as genesis
    import genesis_b200.nn.functional as F
    T, H, I = 512, 256, 384
    g = torch.Generator().manual_seed(3)
    x0 = torch.randn(T, H, generator=g)
    wg0, wu0 = torch.randn(I, H, generator=g) * 0.1, torch.randn(I, H, generator=g) * 0.1
    dy = torch.randn(T, I, generator=g).to(DEV)

    def run(fused):
        x = genesis.Tensor(x0.clone().to(DEV), requires_grad=True)
        wg = genesis.Tensor(wg0.clone().to(DEV), requires_grad=True)
        wu = genesis.Tensor(wu0.clone().to(DEV), requires_grad=True)
        with genesis.amp.autocast(dtype=genesis.bfloat16):
            h = F.linear_swiglu(x, wg, wu) if fused else F.swiglu(F.linear(x, wg), F.linear(x, wu))
        (h * genesis.Tensor(dy.to(h._t.dtype))).sum().backward()
        return h._t.float(), x.grad._t.float(), wg.grad._t.float(), wu.grad._t.float()

    K.reset_fallbacks()
    with K.strict_native(True):
        a = run(True)
    b = run(False)
    for u, v in zip(a, b):
        torch.testing.assert_close(u, v, atol=3e-2 * max(1.0, float(v.abs().max())), rtol=3e-2)
    # fp32 reference for the forward value
    ref = torch.nn.functional.silu(x0 @ wg0.t()) * (x0 @ wu0.t())
    torch.testing.assert_close(a[0].cpu(), ref, atol=0.05, rtol=0.05)
    assert K.fallback_counts() == {}


def test_gemm_routes_large_16_bit_shapes_to_the_pair_kernel():
    before = N.launch_count
    a, b = rnd(4096, 896, dt=torch.bfloat16).to(DEV), rnd(4864, 896, dt=torch.bfloat16, seed=1).to(DEV)
    assert N._pair_width(4096, 4864, 896, N._sms(a.device)) == 256
    assert N._pair_width(4096, 4864, 896, N._sms(a.device), b_mn=1) == 0
    got = N.gemm(a, b)
    check(got, a.float().cpu() @ b.float().cpu().t(), torch.bfloat16, 896)
    assert N.launch_count == before + 1


@pytest.mark.parametrize("M,I,H", [(256, 128, 64), (512, 256, 896), (1000, 448, 200), (2048, 4864, 896)])
def test_pair_gemm_swiglu_backward_epilogue(M, I, H):
    gy = rnd(M, H, dt=torch.bfloat16)
    wd = (rnd(H, I, seed=1) * 0.2).bfloat16()                  # down weight [H, I]
    gu = rnd(M, 2 * I, dt=torch.bfloat16, seed=2)
    dh = gy.float() @ wd.float()
    g, u = gu[:, :I].float(), gu[:, I:].float()
    sg = torch.sigmoid(g)
    ref = torch.cat((dh * u * sg * (1 + g * (1 - sg)), dh * g * sg), 1)
    got = N.dgrad_swiglu_bwd(gy.to(DEV), wd.t().contiguous().to(DEV), gu.to(DEV))
    assert got is not NotImplemented
    check(got, ref, torch.bfloat16, H)


def test_swiglu_mlp_function_with_optimizer_kept_copies():
    """The one-node MLP (activation in the gate|up epilogue, its gradient in the down data-gradient epilogue, K-major
    twins of the weights from the optimizer) against three separate layers."""
    import genesis_b200 as genesis
    import genesis_b200.nn as nn
    import genesis_b200.nn.functional as F
    T, H, I = 512, 256, 384
    g = torch.Generator().manual_seed(5)
    x0 = torch.randn(T, H, generator=g)
    dy = torch.randn(T, H, generator=g).to(DEV)

    def run(fused):
        genesis.manual_seed(1)
        gate, up, down = nn.Linear(H, I, bias=False).cuda(), nn.Linear(H, I, bias=False).cuda(), \
            nn.Linear(I, H, bias=False).cuda()
        params = [gate.weight, up.weight, down.weight]
        opt = genesis.optim.AdamW(params, lr=1e-3)
        opt.enable_shadows(genesis.bfloat16, [[gate.weight, up.weight]], transposed=True)
        x = genesis.Tensor(x0.clone().to(DEV), requires_grad=True)
        with genesis.amp.autocast(dtype=genesis.bfloat16):
            if fused:
                y = F.swiglu_mlp(x, gate.weight, up.weight, down.weight)
            else:
                y = down(F.swiglu(gate(x), up(x)))
        (y * genesis.Tensor(dy.to(y._t.dtype))).sum().backward()
        out = [y._t.float(), x.grad._t.float()] + [p.grad._t.float() for p in params]
        opt.step()                                     # refreshes copies and twins
        opt.disable_shadows()
        return out

    K.reset_fallbacks()
    with K.strict_native(True):
        a = run(True)
    b = run(False)
    for u, v in zip(a, b):
        torch.testing.assert_close(u, v, atol=3e-2 * max(1.0, float(v.abs().max())), rtol=3e-2)
    assert K.fallback_counts() == {}
