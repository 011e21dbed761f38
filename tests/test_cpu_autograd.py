"""Forward values and gradients of every differentiable op against torch.autograd on CPU
(the oracle the reference's own suite uses, `tests/test_functional.py`, with its shape grids)."""
import numpy as np
import pytest
import torch

import genesis_b200 as genesis
import genesis_b200.nn.functional as F

ATOL, RTOL = 1e-5, 1e-5


def mk(*shape, seed=0, pos=False):
    rs = np.random.RandomState(seed + len(shape) + sum(shape))
    a = rs.randn(*shape).astype(np.float32)
    if pos:
        a = np.abs(a) + 0.5
    return a


def pair(a):
    return genesis.tensor(a, requires_grad=True), torch.tensor(a, requires_grad=True)


def check(gfn, tfn, *arrays, atol=ATOL, rtol=RTOL):
    gs, ts = zip(*[pair(a) for a in arrays])
    go, to = gfn(*gs), tfn(*ts)
    np.testing.assert_allclose(go.detach().numpy(), to.detach().numpy(), atol=atol, rtol=rtol)
    w = torch.randn(to.shape, generator=torch.Generator().manual_seed(1))
    (go * genesis.tensor(w.numpy())).sum().backward()
    (to * w).sum().backward()
    for g, t in zip(gs, ts):
        assert g.grad is not None
        np.testing.assert_allclose(g.grad.numpy(), t.grad.numpy(), atol=atol * 10, rtol=rtol * 10)


BCAST = [((4, 5), (4, 5)), ((4, 5), (5,)), ((4, 1), (1, 5)), ((2, 3, 4), (3, 1)), ((1,), (3, 2))]


@pytest.mark.parametrize("sa,sb", BCAST)
def test_binary_ops(sa, sb):
    a, b = mk(*sa), mk(*sb, seed=1, pos=True)
    check(lambda x, y: x + y, lambda x, y: x + y, a, b)
    check(lambda x, y: x - y, lambda x, y: x - y, a, b)
    check(lambda x, y: x * y, lambda x, y: x * y, a, b)
    check(lambda x, y: x / y, lambda x, y: x / y, a, b)
    check(F.maximum, torch.maximum, a, b)


def test_scalar_ops():
    a = mk(3, 4, pos=True)
    check(lambda x: x + 2.0, lambda x: x + 2.0, a)
    check(lambda x: 2.0 - x, lambda x: 2.0 - x, a)
    check(lambda x: x * 3.0, lambda x: x * 3.0, a)
    check(lambda x: 3.0 / x, lambda x: 3.0 / x, a)
    check(lambda x: x / 3.0, lambda x: x / 3.0, a)
    check(lambda x: x ** 3, lambda x: x ** 3, a)
    check(lambda x: x ** 0.5, lambda x: x ** 0.5, a)
    check(lambda x: 2.0 ** x, lambda x: 2.0 ** x, a)
    check(lambda x: -x, lambda x: -x, a)
    check(lambda x, y: x ** y, lambda x, y: x ** y, a, mk(3, 4, seed=2))


@pytest.mark.parametrize("name", ["sin", "cos", "exp", "tanh", "sigmoid", "relu", "abs", "silu", "gelu"])
def test_unary(name):
    a = mk(5, 7)
    tfn = {"silu": torch.nn.functional.silu, "gelu": lambda x: torch.nn.functional.gelu(x, approximate="tanh"),
           "relu": torch.relu, "sigmoid": torch.sigmoid}.get(name, getattr(torch, name, None))
    check(getattr(F, name), tfn, a, atol=1e-5)


def test_log_sqrt_clamp_where():
    a = mk(5, 7, pos=True)
    check(F.log, torch.log, a)
    check(F.sqrt, torch.sqrt, a)
    b = mk(5, 7, seed=3)
    check(lambda x: F.clamp(x, -0.3, 0.5), lambda x: torch.clamp(x, -0.3, 0.5), b)
    cond = b > 0
    check(lambda x, y: F.where(genesis.tensor(cond, dtype=genesis.bool), x, y),
          lambda x, y: torch.where(torch.tensor(cond), x, y), a, b)


REDS = [((1, 1, 1), None), ((5, 3), 0), ((8, 3, 2), 1), ((8, 3, 2), 2), ((8, 3, 64), 1), ((8, 3, 64), 2),
        ((64, 64), 0), ((64, 64), 1), ((32, 32), None), ((1, 64), 0), ((64, 1), 1), ((16, 16, 16), (0, 2))]


@pytest.mark.parametrize("shape,axis", REDS)
def test_reductions(shape, axis):
    a = mk(*shape)
    for keep in (False, True):
        check(lambda x: F.sum(x, axis, keep), lambda x: x.sum() if axis is None and not keep else
              x.sum(dim=axis if axis is not None else tuple(range(x.dim())), keepdim=keep), a)
        check(lambda x: F.mean(x, axis, keep), lambda x: x.mean() if axis is None and not keep else
              x.mean(dim=axis if axis is not None else tuple(range(x.dim())), keepdim=keep), a)
    if axis is None or isinstance(axis, int):
        check(lambda x: F.max(x, axis), lambda x: x.max() if axis is None else x.max(dim=axis)[0], a)
        check(lambda x: F.min(x, axis), lambda x: x.min() if axis is None else x.min(dim=axis)[0], a)
        check(lambda x: F.logsumexp(x, axis), lambda x: torch.logsumexp(x, dim=axis if axis is not None
                                                                        else tuple(range(x.dim()))), a)
    if isinstance(axis, int) and shape[axis] > 1:
        check(lambda x: F.var(x, axis), lambda x: x.var(dim=axis), a)
        check(lambda x: F.std(x, axis), lambda x: x.std(dim=axis), a, atol=1e-4)


MM = [(16, 16, 16), (8, 8, 8), (3, 4, 5), (5, 4, 3), (16, 16, 32), (64, 64, 64), (72, 73, 74), (74, 73, 72)]


@pytest.mark.parametrize("m,n,p", MM)
def test_matmul(m, n, p):
    check(lambda x, y: x @ y, lambda x, y: x @ y, mk(m, n), mk(n, p, seed=1), atol=1e-4)


@pytest.mark.parametrize("b,m,n,p", [(16, 16, 16, 16), (32, 16, 8, 24), (32, 13, 8, 15)])
def test_batched_matmul(b, m, n, p):
    check(lambda x, y: x @ y, lambda x, y: x @ y, mk(b, m, n), mk(b, n, p, seed=1), atol=1e-4)
    check(lambda x, y: x @ y, lambda x, y: x @ y, mk(b, m, n), mk(n, p, seed=1), atol=1e-4)
    check(lambda x, y: x @ y, lambda x, y: x @ y, mk(m, n), mk(b, n, p, seed=1), atol=1e-4)
    check(lambda x, y: x @ y, lambda x, y: x @ y, mk(n), mk(n, p, seed=1), atol=1e-4)
    check(lambda x, y: x @ y, lambda x, y: x @ y, mk(m, n), mk(n, seed=1), atol=1e-4)


def test_shape_ops():
    a = mk(4, 5, 6)
    check(lambda x: x.reshape(20, 6), lambda x: x.reshape(20, 6), a)
    check(lambda x: x.view(4, 30), lambda x: x.reshape(4, 30), a)
    check(lambda x: x.permute(2, 0, 1), lambda x: x.permute(2, 0, 1), a)
    check(lambda x: x.transpose(0, 2), lambda x: x.transpose(0, 2), a)
    check(lambda x: x.T, lambda x: x.permute(2, 1, 0), a)
    check(lambda x: x.unsqueeze(1).squeeze(1), lambda x: x.unsqueeze(1).squeeze(1), a)
    check(lambda x: F.flatten(x, 1), lambda x: x.flatten(1), a)
    check(lambda x: F.broadcast_to(x.unsqueeze(0), (3, 4, 5, 6)), lambda x: x.unsqueeze(0).expand(3, 4, 5, 6), a)
    check(lambda x: x.unsqueeze(0).expand(3, 4, 5, 6), lambda x: x.unsqueeze(0).expand(3, 4, 5, 6), a)
    check(lambda x: x.permute(1, 0, 2).contiguous(), lambda x: x.permute(1, 0, 2).contiguous(), a)
    check(lambda x: F.repeat_interleave(x, 3, dim=1), lambda x: torch.repeat_interleave(x, 3, dim=1), a)


@pytest.mark.parametrize("shape,dim,n", [((5, 5), 0, 1), ((5, 5), 0, 2), ((1, 5, 7), 2, 5)])
def test_stack_cat_split(shape, dim, n):
    arrs = [mk(*shape, seed=i) for i in range(n)]
    check(lambda *xs: F.stack(xs, dim), lambda *xs: torch.stack(xs, dim), *arrs)
    check(lambda *xs: F.cat(xs, dim), lambda *xs: torch.cat(xs, dim), *arrs)
    a = mk(10, 5)
    gx, tx = pair(a)
    gp, tp = F.split(gx, dim=0), torch.split(tx, 1, dim=0)
    assert len(gp) == len(tp)
    (gp[2] * 2 + gp[7]).sum().backward()
    (tp[2] * 2 + tp[7]).sum().backward()
    np.testing.assert_allclose(gx.grad.numpy(), tx.grad.numpy())


def test_getitem_setitem():
    a = mk(4, 5, 6)
    idx = np.array([0, 2, 2, 3])
    check(lambda x: x[1], lambda x: x[1], a)
    check(lambda x: x[1:3, ::2], lambda x: x[1:3, ::2], a)
    check(lambda x: x[..., 2], lambda x: x[..., 2], a)
    check(lambda x: x[:, None, 1], lambda x: x[:, None, 1], a)
    check(lambda x: x[genesis.tensor(idx, dtype=genesis.int64)], lambda x: x[torch.tensor(idx)], a)   # duplicates
    check(lambda x: x[genesis.tensor(idx, dtype=genesis.int64), 1:3], lambda x: x[torch.tensor(idx), 1:3], a)
    r, c = np.array([0, 1, 3]), np.array([4, 0, 2])
    check(lambda x: x[genesis.tensor(r, dtype=genesis.int64), genesis.tensor(c, dtype=genesis.int64)],
          lambda x: x[torch.tensor(r), torch.tensor(c)], a)
    mask = a[:, :, 0] > 0
    check(lambda x: x[genesis.tensor(mask, dtype=genesis.bool)], lambda x: x[torch.tensor(mask)], a)
    gx, tx = pair(a)
    gv, tv = pair(mk(5, 6, seed=9))
    gy, ty = gx * 1.0, tx * 1.0
    gy[1] = gv
    ty[1] = tv
    gy.sum().backward()
    ty.sum().backward()
    np.testing.assert_allclose(gx.grad.numpy(), tx.grad.numpy())
    np.testing.assert_allclose(gv.grad.numpy(), tv.grad.numpy())
    z = genesis.zeros(3, 3)
    z[0, 1] = 5.0
    assert z.numpy()[0, 1] == 5.0


def test_gather_scatter_topk():
    a = mk(6, 7)
    idx = np.random.RandomState(0).randint(0, 7, (6, 3))
    check(lambda x: F.gather(x, 1, genesis.tensor(idx, dtype=genesis.int64)),
          lambda x: torch.gather(x, 1, torch.tensor(idx)), a)
    src = mk(6, 3, seed=4)
    pidx = np.stack([np.random.RandomState(i).permutation(7)[:3] for i in range(6)])
    check(lambda x, s: F.scatter(x, 1, genesis.tensor(pidx, dtype=genesis.int64), s),
          lambda x, s: torch.scatter(x, 1, torch.tensor(pidx), s), a, src)
    check(lambda x, s: F.scatter_add(x, 1, genesis.tensor(idx, dtype=genesis.int64), s),
          lambda x, s: torch.scatter_add(x, 1, torch.tensor(idx), s), a, src)
    check(lambda x: F.topk(x, 3, dim=1)[0], lambda x: torch.topk(x, 3, dim=1)[0], a)
    v, i = F.topk(genesis.tensor(a), 2)
    tv, ti = torch.topk(torch.tensor(a), 2)
    assert np.array_equal(i.numpy(), ti.numpy())
    assert np.array_equal(genesis.argsort(genesis.tensor(a), dim=1).numpy(), torch.argsort(torch.tensor(a), 1).numpy())
    b = genesis.tensor(np.array([1, 3, 3, 0]), dtype=genesis.int64)
    assert genesis.bincount(b, minlength=5).numpy().tolist() == [1, 1, 0, 2, 0]
    assert F.argmax(genesis.tensor(a), 1).numpy().tolist() == torch.tensor(a).argmax(1).tolist()
    oh = F.one_hot(b, 4)
    assert oh.shape == (4, 4) and oh.numpy().sum() == 4


@pytest.mark.parametrize("shape", [(8, 64), (8, 32, 64), (4, 16, 8)])
def test_softmax_ce(shape):
    a = mk(*shape)
    for dim in (-1, 0, 1):
        check(lambda x: F.softmax(x, dim), lambda x: torch.softmax(x, dim), a)
        check(lambda x: F.log_softmax(x, dim), lambda x: torch.log_softmax(x, dim), a)
    logits = mk(16, 10)
    tgt = np.random.RandomState(1).randint(0, 10, (16,))
    tgt_i = tgt.copy()
    tgt_i[3] = -100
    w = np.abs(mk(10, seed=5)) + 0.1
    gt = genesis.tensor(tgt, dtype=genesis.int64)
    for red in ("mean", "sum", "none"):
        check(lambda x: F.cross_entropy(x, gt, reduction=red),
              lambda x: torch.nn.functional.cross_entropy(x, torch.tensor(tgt), reduction=red), logits)
    check(lambda x: F.cross_entropy(x, genesis.tensor(tgt_i, dtype=genesis.int64)),
          lambda x: torch.nn.functional.cross_entropy(x, torch.tensor(tgt_i)), logits)
    check(lambda x: F.cross_entropy(x, gt, weight=torch.tensor(w), reduction="sum"),
          lambda x: torch.nn.functional.cross_entropy(x, torch.tensor(tgt), weight=torch.tensor(w), reduction="sum"),
          logits)


def test_fused_ops_against_composed():
    x, w, b = mk(6, 32), mk(32, seed=1), mk(32, seed=2)
    check(lambda a, ww: F.rms_norm(a, ww, 1e-6),
          lambda a, ww: a * torch.rsqrt(a.pow(2).mean(-1, keepdim=True) + 1e-6) * ww, x, w)
    check(lambda a, ww, bb: F.layer_norm(a, ww, bb, 1e-5),
          lambda a, ww, bb: torch.nn.functional.layer_norm(a, (32,), ww, bb, 1e-5), x, w, b)
    g, u = mk(5, 16), mk(5, 16, seed=3)
    check(F.swiglu, lambda a, c: torch.nn.functional.silu(a) * c, g, u)
    check(lambda a, ww, bb: F.linear(a, ww, bb), torch.nn.functional.linear, mk(3, 7, 32), mk(8, 32, seed=4), mk(8, seed=5),
          atol=1e-4)
    emb, idx = mk(20, 8), np.array([[1, 3, 3], [0, 19, 1]])
    check(lambda ww: F.embedding(ww, genesis.tensor(idx, dtype=genesis.int64)),
          lambda ww: torch.nn.functional.embedding(torch.tensor(idx), ww), emb)


def _torch_rope(x, cos, sin):
    d = x.shape[-1] // 2
    rot = torch.cat((-x[..., d:], x[..., :d]), -1)
    S = x.shape[1]
    return x * cos[:S].reshape(1, S, 1, -1) + rot * sin[:S].reshape(1, S, 1, -1)


@pytest.mark.parametrize("Hq,Hkv,causal", [(4, 4, True), (4, 2, True), (6, 2, False), (3, 1, True)])
def test_rope_and_attention(Hq, Hkv, causal):
    B, S, D = 2, 9, 8
    q, k, v = mk(B, S, Hq, D), mk(B, S, Hkv, D, seed=1), mk(B, S, Hkv, D, seed=2)
    inv = 1.0 / (10000.0 ** (np.arange(0, D, 2) / D))
    fr = np.outer(np.arange(16), inv)
    cos, sin = np.cos(np.concatenate([fr, fr], -1)).astype(np.float32), np.sin(np.concatenate([fr, fr], -1)).astype(np.float32)
    check(lambda a: F.rope(a, genesis.tensor(cos), genesis.tensor(sin)),
          lambda a: _torch_rope(a, torch.tensor(cos), torch.tensor(sin)), q)

    def tattn(a, b, c):
        g = Hq // Hkv
        at, bt, ct = (t.permute(0, 2, 1, 3) for t in (a, b.repeat_interleave(g, 2), c.repeat_interleave(g, 2)))
        return torch.nn.functional.scaled_dot_product_attention(at, bt, ct, is_causal=causal).permute(0, 2, 1, 3)
    check(lambda a, b, c: F.flash_attention(a, b, c, causal=causal), tattn, q, k, v, atol=1e-5)


def test_hooks_no_grad_inplace_rules():
    x = genesis.tensor(mk(3, 3), requires_grad=True)
    seen = []
    y = x * 2
    y.register_hook(lambda g: seen.append("mid") or g * 3)
    x.register_hook(lambda g: seen.append("leaf"))
    x.register_post_accumulate_grad_hook(lambda t: seen.append("post"))
    y.sum().backward()
    assert seen == ["mid", "leaf", "post"]
    np.testing.assert_allclose(x.grad.numpy(), np.full((3, 3), 6.0, np.float32))
    with genesis.no_grad():
        z = x * 2
    assert not z.requires_grad and z.creator is None
    with pytest.raises(RuntimeError):
        x += 1.0
    d = x.detach()
    d += 1.0
    assert genesis.is_grad_enabled()

    @genesis.no_grad()
    def f(t):
        return t * 2
    assert not f(x).requires_grad


def test_gradient_routing_with_non_grad_first_input():
    # an earlier input that needs no gradient must not shift the gradients of the later ones
    a = genesis.tensor(mk(4, 3))
    w = genesis.tensor(mk(3, 5, seed=1), requires_grad=True)
    (a @ w).sum().backward()
    assert w.grad.shape == (3, 5)
    np.testing.assert_allclose(w.grad.numpy(), np.repeat(mk(4, 3).sum(0)[:, None], 5, 1), rtol=1e-5)
    c = genesis.tensor(mk(4, 3, seed=2))
    m = genesis.tensor(mk(4, 3, seed=3), requires_grad=True)
    (c * m).sum().backward()
    np.testing.assert_allclose(m.grad.numpy(), mk(4, 3, seed=2))


def test_custom_function_tensor_api():
    class Square(genesis.Function):
        @staticmethod
        def forward(ctx, a):
            ctx.save_for_backward(a)
            return a * a

        @staticmethod
        def backward(ctx, g):
            (a,) = ctx.saved_tensors
            return g * a * 2.0
    x = genesis.tensor(mk(4), requires_grad=True)
    Square.apply(x).sum().backward()
    np.testing.assert_allclose(x.grad.numpy(), 2 * mk(4), rtol=1e-6)


def test_tensor_basics():
    t = genesis.tensor([1, 2, 3])
    assert t.dtype == genesis.float32 and t.dtype == "float32"
    assert genesis.from_numpy(np.arange(3)).dtype == genesis.int64
    assert genesis.from_numpy(np.arange(3, dtype=np.int32)).dtype == genesis.int32
    assert genesis.from_numpy(np.float64(2.0)).shape == ()
    assert genesis.arange(5).dtype == genesis.int64 and genesis.arange(0, 1, 0.25).dtype == genesis.float32
    assert genesis.eye(3).numpy().trace() == 3
    b = genesis.ones(2, 2, dtype=genesis.bfloat16)
    assert b.numpy().dtype == np.float32 and b.element_size() == 2
    with pytest.raises(RuntimeError):
        genesis.ones(2, requires_grad=True).numpy()
    assert genesis.tensor(2.5).item() == 2.5 and float(genesis.tensor(2.5)) == 2.5
    assert genesis.device("cuda:1").index == 1 and genesis.device("cpu").is_cpu()
    assert genesis.zeros(2, 3).to("float16").dtype == genesis.float16
    assert len(genesis.zeros(4, 2)) == 4
    genesis.manual_seed(3)
    a = genesis.randn(4).numpy()
    genesis.manual_seed(3)
    assert np.array_equal(a, genesis.randn(4).numpy())
    assert genesis.allclose(genesis.ones(3), genesis.ones(3))


def test_post_accumulate_hook_fires_once_for_a_tensor_used_twice():
    import genesis_b200 as genesis
    w = genesis.Tensor(torch.tensor([1.0, 2.0, 3.0]), requires_grad=True)
    seen = []
    w.register_post_accumulate_grad_hook(lambda t: seen.append(t.grad._t.clone()))
    x = genesis.Tensor(torch.tensor([2.0, 2.0, 2.0]))
    ((w * x).sum() + (w * w).sum()).backward()
    assert len(seen) == 1                                       # one call, with the complete gradient
    assert torch.allclose(seen[0], torch.tensor([2.0 + 2.0, 2.0 + 4.0, 2.0 + 6.0]))


def test_reference_export_names_exist_and_work():
    import genesis_b200 as genesis
    import genesis_b200.nn.functional as F
    from genesis_b200.function import AMPPolicy
    x = genesis.Tensor(torch.tensor([3.0, 4.0]), requires_grad=True)
    n = F.norm(x)
    n.backward()
    assert abs(float(n.item()) - 5.0) < 1e-6 and torch.allclose(x.grad._t, torch.tensor([0.6, 0.8]))
    assert F.View is F.Reshape and F.GetItemView is F.GetItem
    assert F.Equal.apply(x, x)._t.all() and int(F.Argmax.apply(x)._t) == 1 and int(F.Argmin.apply(x)._t) == 0
    assert F.cast_to_fp16(x).dtype == genesis.float16 and F.cast_fp32(F.cast_to_fp16(x)).dtype == genesis.float32
    assert F.sum_to_shape(genesis.Tensor(torch.ones(3, 4)), (1, 4))._t.tolist() == [[3.0] * 4]
    assert genesis.amp.get_amp_dtype(AMPPolicy.FP32) == genesis.float32
    assert genesis.amp.get_amp_dtype(AMPPolicy.PRESERVE, x) is None
    assert genesis.amp.get_amp_dtype(AMPPolicy.PROMOTE, x, F.cast_to_fp16(x)) == genesis.float32
    assert isinstance(genesis.amp.get_amp_cache(), dict)
    assert genesis.cuda.get_memory_manager(0).device == 0


def test_fused_qkv_projection_and_rope_match_the_separate_ops():
    import genesis_b200 as genesis
    import genesis_b200.nn.functional as F
    torch.manual_seed(0)
    B, S, Hd, Hq, Hkv, D = 2, 5, 24, 4, 2, 8
    def leaf(*shape):
        return genesis.Tensor(torch.randn(*shape), requires_grad=True)
    x1, x2 = leaf(B, S, Hd), None
    x2 = genesis.Tensor(x1._t.clone(), requires_grad=True)
    ws = [leaf(Hq * D, Hd), leaf(Hkv * D, Hd), leaf(Hkv * D, Hd)]
    bs = [leaf(Hq * D), leaf(Hkv * D), leaf(Hkv * D)]
    ws2 = [genesis.Tensor(w._t.clone(), requires_grad=True) for w in ws]
    bs2 = [genesis.Tensor(b._t.clone(), requires_grad=True) for b in bs]
    pos = torch.arange(16).float()[:, None] * (1.0 / 10000 ** (torch.arange(0, D, 2).float() / D))[None]
    cos, sin = torch.cat((pos.cos(), pos.cos()), -1), torch.cat((pos.sin(), pos.sin()), -1)
    gcos, gsin = genesis.Tensor(cos), genesis.Tensor(sin)
    # fused path
    y = F.fused_linear(x1, ws, bs)
    q, k, v = F.qkv_rope(y, gcos, gsin, None, Hq, Hkv, D)
    # separate path
    q2 = F.rope(F.reshape(F.linear(x2, ws2[0], bs2[0]), (B, S, Hq, D)), gcos, gsin)
    k2 = F.rope(F.reshape(F.linear(x2, ws2[1], bs2[1]), (B, S, Hkv, D)), gcos, gsin)
    v2 = F.reshape(F.linear(x2, ws2[2], bs2[2]), (B, S, Hkv, D))
    for a, b in ((q, q2), (k, k2), (v, v2)):
        assert torch.allclose(a._t, b._t, atol=1e-5)
    gq, gk, gv = torch.randn_like(q._t), torch.randn_like(k._t), torch.randn_like(v._t)
    ((q * genesis.Tensor(gq)).sum() + (k * genesis.Tensor(gk)).sum() + (v * genesis.Tensor(gv)).sum()).backward()
    ((q2 * genesis.Tensor(gq)).sum() + (k2 * genesis.Tensor(gk)).sum() + (v2 * genesis.Tensor(gv)).sum()).backward()
    assert torch.allclose(x1.grad._t, x2.grad._t, atol=1e-4)
    for a, b in zip(ws + bs, ws2 + bs2):
        assert torch.allclose(a.grad._t, b.grad._t, atol=1e-4)


def test_fused_gate_up_swiglu_matches_the_separate_ops():
    import genesis_b200 as genesis
    import genesis_b200.nn.functional as F
    torch.manual_seed(1)
    x1 = genesis.Tensor(torch.randn(3, 7, 16), requires_grad=True)
    x2 = genesis.Tensor(x1._t.clone(), requires_grad=True)
    wg, wu = (genesis.Tensor(torch.randn(24, 16) * 0.3, requires_grad=True) for _ in range(2))
    wg2, wu2 = genesis.Tensor(wg._t.clone(), requires_grad=True), genesis.Tensor(wu._t.clone(), requires_grad=True)
    h1 = F.swiglu_fused(F.fused_linear(x1, [wg, wu]))
    h2 = F.swiglu(F.linear(x2, wg2), F.linear(x2, wu2))
    assert torch.allclose(h1._t, h2._t, atol=1e-5)
    go = torch.randn_like(h1._t)
    (h1 * genesis.Tensor(go)).sum().backward()
    (h2 * genesis.Tensor(go)).sum().backward()
    assert torch.allclose(x1.grad._t, x2.grad._t, atol=1e-4)
    assert torch.allclose(wg.grad._t, wg2.grad._t, atol=1e-4) and torch.allclose(wu.grad._t, wu2.grad._t, atol=1e-4)


def test_small_reference_names_exist_and_work():
    """Helpers the reference exposes beside its main API: dtype lists, cast helpers, `check_dtype`, a hand-built
    `AccumulateGrad`, `nn.utils.norm`, the profiling table."""
    import genesis_b200.function as Fn
    import genesis_b200.nn as gnn
    from genesis_b200 import dtypes
    import importlib
    prof = importlib.import_module("genesis_b200.utils.profile")
    assert genesis.bfloat16 in dtypes.floating_dtypes and genesis.int64 in dtypes.integer_dtypes
    assert len(dtypes.all_dtypes) == 10 and dtypes.bool not in dtypes.integer_dtypes
    x = genesis.tensor([[1.0, -2.0], [3.0, 4.0]], requires_grad=True)
    h = Fn.cast_to_bf16(x)
    assert h.dtype == genesis.bfloat16 and Fn.cast_to_bf16(h) is h and Fn.cast_to_fp32(x) is x
    assert Fn.check_dtype({"a": [h]}, genesis.bfloat16) and not Fn.check_dtype((x,), genesis.float16)
    n = gnn.utils.norm(x)
    assert abs(float(n.item()) - 30.0 ** 0.5) < 1e-5
    n.backward()
    assert torch.allclose(x.grad._t, x._t / 30.0 ** 0.5, atol=1e-6)
    leaf = genesis.tensor([1.0, 2.0], requires_grad=True)
    node = Fn.AccumulateGrad(leaf)
    node.apply_grad(genesis.tensor([0.5, 0.5]))
    node.apply_grad(genesis.tensor([0.5, 0.5]))
    assert leaf.grad._t.tolist() == [1.0, 1.0]

    @prof.profile_method
    def f(a):
        return a + 1
    f(1)
    f(2)
    key = [k for k in prof.profile_data if k.endswith("f")][0]
    assert prof.profile_data[key]["calls"] == 2 and prof.profile_data[key]["total_time"] >= 0.0
    prof.print_profile_data()


def test_add_rms_norm_equals_separate_add_and_norm():
    """(x + r, rms_norm(x + r)) as one op gives the values and gradients of the two separate ops, also when only
    one of its outputs is used; a dense block run with deferred additions equals the plain block."""
    import genesis_b200.nn as gnn
    import genesis_b200.nn.functional as F
    g = torch.Generator().manual_seed(0)
    xv, rv, wv = torch.randn(5, 7, 16, generator=g), torch.randn(5, 7, 16, generator=g), torch.rand(16, generator=g) + 0.5
    for use in ("both", "sum", "norm"):
        ts = []
        for fused in (False, True):
            x, r = genesis.Tensor(xv.clone(), requires_grad=True), genesis.Tensor(rv.clone(), requires_grad=True)
            w = genesis.Tensor(wv.clone(), requires_grad=True)
            if fused:
                s, y = F.add_rms_norm(x, r, w, 1e-6)
            else:
                s = x + r
                y = F.rms_norm(s, w, 1e-6)
            loss = 0
            if use in ("both", "sum"):
                loss = loss + (s * s).sum()
            if use in ("both", "norm"):
                loss = loss + (y * 3.0).sum() + (y * y).sum()
            loss.backward()
            ts.append((s._t, y._t, x.grad._t, r.grad._t, None if w.grad is None else w.grad._t))
        for a, b in zip(*ts):
            assert (a is None and b is None) or torch.allclose(a, b, atol=1e-5, rtol=1e-5)
    from genesis_b200.models.transformers import TransformerConfig
    from genesis_b200.models.transformers.dense import TransformerBlock
    genesis.manual_seed(1)
    cfg = TransformerConfig(vocab_size=64, hidden_size=32, intermediate_size=64, num_hidden_layers=1,
                            num_attention_heads=4, num_key_value_heads=2, head_dim=8, max_position_embeddings=32)
    blk = TransformerBlock(cfg)
    x = genesis.Tensor(torch.randn(2, 9, 32, generator=g))
    b0 = genesis.Tensor(torch.randn(2, 9, 32, generator=g))
    with genesis.no_grad():
        want = blk(x + b0)
        stream, branch = blk.forward_deferred(x, b0)
        first, fb = blk.forward_deferred(x + b0, None)
    assert torch.allclose((stream + branch)._t, want._t, atol=1e-5)
    assert torch.allclose((first + fb)._t, want._t, atol=1e-5)
    norm = gnn.RMSNorm(32)
    assert norm.add_forward(x)[0] is x


def test_embedding_gradient_scatters_into_existing_gradient():
    """The embedding gradient reaches its leaf as (indices, rows): alone it becomes a dense tensor, with a tied
    output projection or across two backward passes it is scattered into the gradient that is already there, and a
    tensor hook still sees a dense gradient.  All equal to torch's dense result."""
    import genesis_b200.nn.functional as F
    g = torch.Generator().manual_seed(2)
    wv = torch.randn(11, 6, generator=g)
    idx = torch.tensor([[1, 3, 3], [10, 1, 0]])
    tw = wv.clone().requires_grad_(True)
    (torch.nn.functional.embedding(idx, tw).sum(1) @ tw.t()).pow(2).sum().backward()
    ref_tied = tw.grad.clone()
    tw.grad = None
    torch.nn.functional.embedding(idx, tw).pow(2).sum().backward()
    ref_alone = tw.grad.clone()

    w = genesis.Tensor(wv.clone(), requires_grad=True)
    (F.embedding(w, genesis.Tensor(idx)) ** 2).sum().backward()
    assert torch.allclose(w.grad._t, ref_alone, atol=1e-5)
    # second backward pass accumulates by scattering in place
    (F.embedding(w, genesis.Tensor(idx)) ** 2).sum().backward()
    assert torch.allclose(w.grad._t, 2 * ref_alone, atol=1e-5)
    # tied: lookup and output projection share the weight
    w2 = genesis.Tensor(wv.clone(), requires_grad=True)
    seen = []
    h = F.embedding(w2, genesis.Tensor(idx)).sum(1)
    ((h @ w2.transpose(0, 1)) ** 2).sum().backward()
    assert torch.allclose(w2.grad._t, ref_tied, atol=1e-4)
    # with a hook the gradient contributions arrive dense
    w3 = genesis.Tensor(wv.clone(), requires_grad=True)
    w3.register_hook(lambda gr: seen.append(tuple(gr.shape)) or gr)
    (F.embedding(w3, genesis.Tensor(idx)) ** 2).sum().backward()
    assert seen == [(11, 6)] and torch.allclose(w3.grad._t, ref_alone, atol=1e-5)


def test_linear_weight_gradient_goes_straight_into_a_preallocated_slot():
    """A weight with a gradient slot (`_grad_buf`, what DDP hands out) gets its gradient written by the weight-gradient
    product itself: overwritten when the weight has no gradient yet (stale slot contents do not matter), accumulated
    when its gradient already lives there, shared use in two layers included; a tensor hook falls back to the copy."""
    import genesis_b200.nn as gnn
    import genesis_b200.nn.functional as F
    g = torch.Generator().manual_seed(4)
    xv = torch.randn(5, 8, generator=g)
    lin = gnn.Linear(8, 6, bias=True)
    ref_w = lin.weight._t.clone().requires_grad_(True)
    ref_b = lin.bias._t.clone().requires_grad_(True)
    (torch.nn.functional.linear(xv, ref_w, ref_b) ** 2).sum().backward()
    want = ref_w.grad.clone()
    slot = torch.full((6, 8), 123.0)                               # stale values must be overwritten
    lin.weight._grad_buf = slot
    (lin(genesis.Tensor(xv)) ** 2).sum().backward()
    assert lin.weight.grad._t.data_ptr() == slot.data_ptr()
    assert torch.allclose(slot, want, atol=1e-5)
    (lin(genesis.Tensor(xv)) ** 2).sum().backward()              # second pass accumulates in the slot
    assert lin.weight.grad._t.data_ptr() == slot.data_ptr() and torch.allclose(slot, 2 * want, atol=1e-5)
    # the same weight in two layers of one graph
    lin.weight.grad = None
    y = F.linear(F.linear(genesis.Tensor(xv), lin.weight)[:, :6] @ genesis.Tensor(torch.eye(6, 8)), lin.weight)
    (y ** 2).sum().backward()
    w2 = lin.weight._t.clone().requires_grad_(True)
    t = torch.nn.functional.linear(torch.nn.functional.linear(xv, w2)[:, :6] @ torch.eye(6, 8), w2)
    (t ** 2).sum().backward()
    assert lin.weight.grad._t.data_ptr() == slot.data_ptr() and torch.allclose(slot, w2.grad, atol=1e-4)
    # hooks see the gradient first, so it cannot be produced in place
    lin.weight.grad = None
    lin.weight.register_hook(lambda gr: gr * 2.0)
    (lin(genesis.Tensor(xv)) ** 2).sum().backward()
    assert torch.allclose(lin.weight.grad._t, 2 * want, atol=1e-5)


def test_fused_projection_gradient_goes_straight_into_adjacent_slots():
    """Weights of a fused projection whose gradient slots lie back to back (as DDP lays them out) receive their
    gradients from one weight-gradient product writing through a stacked view; slots that are not adjacent fall
    back to the copy."""
    import genesis_b200.nn.functional as F
    g = torch.Generator().manual_seed(5)
    xv = torch.randn(7, 8, generator=g)
    ws = [torch.randn(n, 8, generator=g) for n in (6, 2, 2)]
    refs = [w.clone().requires_grad_(True) for w in ws]
    (torch.cat([torch.nn.functional.linear(xv, r) for r in refs], -1) ** 2).sum().backward()
    for adjacent in (True, False):
        flat = torch.full((10 * 8 + 16,), 7.0)
        offs = (0, 48, 64) if adjacent else (0, 56, 80)
        params = [genesis.Tensor(w.clone(), requires_grad=True) for w in ws]
        for p, o in zip(params, offs):
            p._grad_buf = flat[o:o + p._t.numel()].view(p._t.shape)
        (F.fused_linear(genesis.Tensor(xv), params) ** 2).sum().backward()
        for p, r in zip(params, refs):
            assert p.grad._t.data_ptr() == p._grad_buf.data_ptr()
            assert torch.allclose(p.grad._t, r.grad, atol=1e-4)
        # second pass accumulates
        (F.fused_linear(genesis.Tensor(xv), params) ** 2).sum().backward()
        for p, r in zip(params, refs):
            assert torch.allclose(p._grad_buf, 2 * r.grad, atol=1e-4)
