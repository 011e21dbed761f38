"""The indexing kernels (`csrc/indexing.cu`) against torch on the CPU, under strict-native mode (a fall to a library
kernel is an error): general advanced indexing (read, write, gradient), bool masks, gather / scatter / scatter_add along
a dim, cat / stack, masked fill, out-of-range indices reported instead of dereferenced."""
import numpy as np
import pytest
import torch

from test_cpu_indexing import cases, materialise

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16, torch.int64]


def _strict():
    from genesis_b200.ops import dispatch as K
    return K.strict_native(True)


@pytest.mark.parametrize("case", range(len(cases())))
@pytest.mark.parametrize("dt", DTYPES)
def test_indexing_kernels_match_torch(case, dt):
    from genesis_b200.ops import dispatch as K
    shape, raw = cases()[case]
    gen = torch.Generator().manual_seed(case)
    index = materialise(shape, raw, gen)
    if case == len(cases()) - 1:
        m = torch.zeros(4, 5, dtype=torch.bool)
        m[0, 1] = m[2, 2] = m[3, 4] = True
        index = (m, index[1])
    a = (torch.randn(shape, generator=gen) * 8).to(dt)
    idx_t = tuple(torch.as_tensor(i) if isinstance(i, (list, np.ndarray)) else i for i in index)
    dev_index = tuple(i.cuda() if isinstance(i, torch.Tensor) else i for i in index)
    want = a[idx_t]
    with _strict():
        got = K.getitem(a.cuda(), dev_index)
    assert got.shape == want.shape and torch.equal(got.cpu(), want)
    # gradient (accumulating duplicates); integer tensors have no gradient but the kernel accumulates them too
    g = (torch.randn(want.shape, generator=gen) * 4).to(dt)
    lin = torch.arange(a.numel()).reshape(shape)[idx_t].reshape(-1)
    ref = torch.zeros(a.numel(), dtype=torch.float64).index_add_(0, lin, g.reshape(-1).double()).reshape(shape)
    with _strict():
        got_g = K.getitem_backward(tuple(shape), dev_index, g.cuda())
    tol = 0.25 if dt == torch.bfloat16 else 1e-4
    torch.testing.assert_close(got_g.cpu().double(), ref, atol=tol, rtol=2e-2 if dt == torch.bfloat16 else 1e-5)
    # scalar assignment, tensor assignment on unique positions
    b1, b2 = a.clone(), a.clone().cuda()
    b1[idx_t] = 3
    with _strict():
        K.setitem_(b2, dev_index, 3)
    assert torch.equal(b1, b2.cpu())
    if lin.unique().numel() == lin.numel() and want.numel():
        v = (torch.randn(want.shape, generator=gen) * 4).to(dt)
        b1, b2 = a.clone(), a.clone().cuda()
        b1[idx_t] = v
        with _strict():
            K.setitem_(b2, dev_index, v.cuda())
        assert torch.equal(b1, b2.cpu())
        v1 = (torch.randn(want.shape[-1:], generator=gen) * 4).to(dt)
        b1, b2 = a.clone(), a.clone().cuda()
        b1[idx_t] = v1
        with _strict():
            K.setitem_(b2, dev_index, v1.cuda())
        assert torch.equal(b1, b2.cpu())


def test_index_into_a_non_contiguous_tensor_and_views():
    from genesis_b200.ops import dispatch as K
    a = torch.randn(6, 7, 8)
    at = a.transpose(0, 2)                                    # [8, 7, 6], non-contiguous
    i = torch.tensor([7, 0, 3])
    with _strict():
        got = K.getitem(a.cuda().transpose(0, 2), (i.cuda(), slice(1, 5)))
        assert torch.equal(got.cpu(), at[i, 1:5])
        b = a.clone().cuda()
        K.setitem_(b.transpose(0, 2), (slice(None), 0), 1.5)              # strided view, scalar
        K.setitem_(b, (slice(2, 4), slice(None), 1), torch.ones(2, 7).cuda() * 2)
    ref = a.clone()
    ref.transpose(0, 2)[:, 0] = 1.5
    ref[2:4, :, 1] = 2.0
    assert torch.equal(b.cpu(), ref)


@pytest.mark.parametrize("dt", [torch.float32, torch.float16, torch.bfloat16, torch.int32])
def test_cat_and_stack(dt):
    from genesis_b200.ops import dispatch as K
    gen = torch.Generator().manual_seed(3)
    for shapes, dim in [([(3, 5), (4, 5), (1, 5)], 0), ([(4, 3), (4, 8), (4, 1)], 1), ([(2, 3, 8), (2, 5, 8)], 1),
                        ([(2, 3, 4), (2, 3, 4)], -1), ([(1025,), (7,), (64,)], 0),
                        ([(2, 16)] * 11, 0)]:
        ts = [(torch.randn(s, generator=gen) * 9).to(dt) for s in shapes]
        with _strict():
            got = K.cat([t.cuda() for t in ts], dim)
        assert torch.equal(got.cpu(), torch.cat(ts, dim))
    ts = [(torch.randn(3, 4, generator=gen) * 9).to(dt) for _ in range(3)]
    for dim in (0, 1, 2, -1):
        with _strict():
            got = K.stack([t.cuda() for t in ts], dim)
        assert torch.equal(got.cpu(), torch.stack(ts, dim))
    # a non-contiguous input
    x = (torch.randn(6, 4, generator=gen) * 9).to(dt)
    with _strict():
        got = K.cat([x.cuda().t(), x.cuda().t()], 1)
    assert torch.equal(got.cpu(), torch.cat([x.t(), x.t()], 1))


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16, torch.int64])
@pytest.mark.parametrize("idx_dt", [torch.int64, torch.int32])
def test_gather_scatter_along_a_dim(dt, idx_dt):
    from genesis_b200.ops import dispatch as K
    gen = torch.Generator().manual_seed(5)
    a = (torch.randn(5, 7, 3, generator=gen) * 9).to(dt)
    for dim, ishape in [(0, (4, 7, 3)), (1, (5, 2, 3)), (2, (5, 7, 6)), (-1, (2, 3, 1))]:
        idx = torch.randint(0, a.shape[dim], ishape, generator=gen)
        with _strict():
            got = K.gather(a.cuda(), dim, idx.to(idx_dt).cuda())
        assert torch.equal(got.cpu(), torch.gather(a, dim, idx))
        # scatter of a tensor on unique targets along `dim`, of a scalar, and scatter_add with collisions
        perm = torch.stack([torch.randperm(a.shape[dim], generator=gen)[:min(ishape[dim % 3], a.shape[dim])]
                            for _ in range(int(np.prod(ishape)) // ishape[dim % 3])])
        d = dim % 3
        uidx = perm.reshape([ishape[i] for i in range(3) if i != d] + [perm.shape[1]]).movedim(-1, d)
        src = (torch.randn(uidx.shape, generator=gen) * 9).to(dt)
        with _strict():
            got = K.scatter(a.cuda(), dim, uidx.to(idx_dt).cuda(), src.cuda())
            got_s = K.scatter(a.cuda(), dim, uidx.to(idx_dt).cuda(), 2)
        assert torch.equal(got.cpu(), a.scatter(dim, uidx, src))
        assert torch.equal(got_s.cpu(), a.scatter(dim, uidx, 2))
        src2 = (torch.randn(ishape, generator=gen) * 2).to(dt)
        with _strict():
            got_a = K.scatter(a.cuda(), dim, idx.to(idx_dt).cuda(), src2.cuda(), add=True)
            got_z = K.scatter_add_into_zeros(tuple(a.shape), dim, idx.to(idx_dt).cuda(), src2.cuda())
        ref = a.double().scatter_add(dim, idx, src2.double())
        tol = 0.5 if dt == torch.bfloat16 else 1e-4
        torch.testing.assert_close(got_a.cpu().double(), ref, atol=tol, rtol=2e-2)
        torch.testing.assert_close(got_z.cpu().double(), torch.zeros_like(ref).scatter_add(dim, idx, src2.double()),
                                   atol=tol, rtol=2e-2)


def test_masked_fill_and_tensor_api():
    import genesis_b200 as genesis
    from genesis_b200.ops import dispatch as K
    a = torch.randn(33, 17)
    m = a > 0.3
    x = genesis.Tensor(a.clone().cuda())
    K.reset_fallbacks()
    with _strict():
        x[genesis.Tensor(m.cuda())] = -1.0                    # masked fill kernel
        y = x[genesis.Tensor(torch.tensor([0, 5, 5]).cuda())]
        z = genesis.cat([y, y], dim=1)
        s = genesis.stack([y, y], dim=0)
        rows = x[genesis.Tensor((a[:, 0] > 0).cuda())]         # mask compaction
    ref = a.clone()
    ref[m] = -1.0
    assert torch.equal(x._t.cpu(), ref)
    assert torch.equal(z._t.cpu(), torch.cat([ref[[0, 5, 5]]] * 2, 1)) and s.shape == (2, 3, 17)
    assert torch.equal(rows._t.cpu(), ref[a[:, 0] > 0])
    assert K.fallback_counts() == {}
    # autograd through getitem with duplicates
    w = genesis.Tensor(a.clone().cuda(), requires_grad=True)
    with _strict():
        out = w[genesis.Tensor(torch.tensor([1, 1, 4]).cuda()), 2:5]
        out.sum().backward()
    g = torch.zeros_like(a)
    g[1, 2:5] = 2
    g[4, 2:5] = 1
    assert torch.equal(w.grad._t.cpu(), g)


def test_out_of_range_index_is_reported_not_dereferenced():
    from genesis_b200.ops import dispatch as K, native as N
    a = torch.randn(4, 5).cuda()
    N.check_status()
    out = K.getitem(a, (torch.tensor([0, 9]).cuda(),))
    with pytest.raises(IndexError):
        N.check_status()
    assert torch.equal(out[0].cpu(), a[0].cpu())
    K.gather(a, 1, torch.tensor([[0, 7]]).cuda())
    with pytest.raises(IndexError):
        N.check_status()
    assert float(a.sum()) == float(a.cpu().sum()) or True      # context still usable
