"""The index planner (`genesis_b200.ops.indexing`) against torch's own indexing, with the tensor-index stage emulated
in torch (`emulate=True`): every case checks the result of `a[index]`, of `a[index] = value` and of the gradient of
`a[index]`.  The same case grid runs on the GPU kernels in `tests/test_gpu_indexing.py`.
Case grid after the reference's `tests/test_functional.py:650-1128`."""
import numpy as np
import pytest
import torch

from genesis_b200.ops import indexing


def cases():
    L = torch.tensor
    return [
        ((5, 6), (2,)),
        ((5, 6), (slice(1, 4),)),
        ((5, 6), (slice(None), 3)),
        ((5, 6), (slice(None, None, 2), slice(1, None, 2))),
        ((4, 5, 6), (Ellipsis, 2)),
        ((4, 5, 6), (None, 1, Ellipsis, None)),
        ((5, 6), (L([0, 2, 4]),)),
        ((5, 6), (L([4, 0, 0, 3]), L([1, 1, 5, 2]))),                    # two index tensors, duplicates
        ((5, 6), (slice(None), L([0, 5, 5]))),                           # column gather
        ((4, 5, 6), (L([[0, 1], [3, 3]]),)),                             # 2-D index
        ((4, 5, 6), (slice(None), L([0, 4]), slice(None))),
        ((4, 5, 6), (slice(1, 3), L([0, 4]), L([[5], [0]]))),            # broadcasting index tensors, pre dims
        ((4, 5, 6), (L([0, 3]), slice(None), L([1, 2]))),                # non-adjacent: broadcast block first
        ((4, 5, 6), (0, slice(None), L([1, 2, 2]))),                     # int counts as advanced (non-adjacent)
        ((4, 5, 6), (L([1, 2]), 0)),
        ((4, 5, 6), (slice(None), 0, L([1, 2]))),
        ((4, 5, 6), (L([-1, -4]), L([-5, 0]))),                          # negative indices
        ((4, 5, 6), (L([0, 1], dtype=torch.int32),)),
        ((4, 5, 6), (None, L([0, 1]))),
        ((4, 5, 6), (L([0, 1]), None, L([2, 3]))),
        ((2, 3, 2, 3, 2, 3), (slice(None), slice(None), slice(None), slice(None), L([0, 1, 1]))),   # long pre side
        ((5, 6), ([0, 2],)),                                             # python list
        ((5, 6), (np.array([1, 3]),)),
        ((5, 6), ("mask", (5,))),                                        # mask over the leading dim
        ((5, 6), ("mask", (5, 6))),                                      # full mask
        ((4, 5, 6), (slice(None), "mask", (5,))),                        # mask in the middle
        ((4, 5, 6), (slice(None), "mask", (5, 6))),
        ((4, 5, 6), ("mask", (4, 5), L([0, 1, 2]))),                     # handled below (needs matching count)
    ]


def materialise(shape, index, gen):
    out, it = [], iter(index)
    for item in it:
        if isinstance(item, str):
            mshape = next(it)
            m = torch.rand(mshape, generator=gen) > 0.5
            m.reshape(-1)[0] = True
            out.append(m)
        else:
            out.append(item)
    return tuple(out)


@pytest.mark.parametrize("case", range(len(cases())))
def test_planner_matches_torch(case):
    shape, raw = cases()[case]
    gen = torch.Generator().manual_seed(case)
    index = materialise(shape, raw, gen)
    if case == len(cases()) - 1:
        # a mask and an index tensor broadcast together: make the counts agree
        m = torch.zeros(4, 5, dtype=torch.bool)
        m[0, 1] = m[2, 2] = m[3, 4] = True
        index = (m, index[1])
    a = torch.randn(shape, generator=gen)
    want = a[index]
    got = indexing.getitem(a, index, emulate=True)
    assert got is not NotImplemented
    assert got.shape == want.shape and torch.equal(got, want)
    # gradient: zeros + accumulate
    g = torch.randn(want.shape, generator=gen)
    ref = torch.zeros_like(a)
    idx_t = tuple(torch.as_tensor(i) if isinstance(i, (list, np.ndarray)) else i for i in index)
    lin = torch.arange(a.numel()).reshape(shape)[idx_t].reshape(-1)
    ref.reshape(-1).index_add_(0, lin, g.reshape(-1))
    got_g = indexing.getitem_backward(shape, index, g, emulate=True)
    assert got_g is not NotImplemented
    torch.testing.assert_close(got_g, ref)
    # assignment of a tensor and of a scalar (unique positions only matter: compare where torch is deterministic)
    b1, b2 = a.clone(), a.clone()
    b1[idx_t] = 7.5
    assert indexing.setitem_(b2, index, 7.5, emulate=True) is b2
    assert torch.equal(b1, b2)
    uniq = lin.unique().numel() == lin.numel()
    if uniq and want.numel():
        v = torch.randn(want.shape, generator=gen)
        b1, b2 = a.clone(), a.clone()
        b1[idx_t] = v
        indexing.setitem_(b2, index, v, emulate=True)
        assert torch.equal(b1, b2)
        # broadcast value
        v1 = torch.randn(want.shape[-1:], generator=gen)
        b1, b2 = a.clone(), a.clone()
        b1[idx_t] = v1
        indexing.setitem_(b2, index, v1, emulate=True)
        assert torch.equal(b1, b2)


def test_planner_errors_and_limits():
    a = torch.randn(3, 4)
    with pytest.raises(IndexError):
        indexing.getitem(a, (0, 0, 0), emulate=True)
    with pytest.raises(IndexError):
        indexing.getitem(a, (torch.tensor([0.5]),), emulate=True)
    with pytest.raises(IndexError):
        indexing.getitem(a, (torch.ones(2, 4, dtype=torch.bool),), emulate=True)
    with pytest.raises(IndexError):
        indexing.getitem(a, (torch.tensor([0, 1]), torch.tensor([0, 1, 2])), emulate=True)
    five = tuple(torch.tensor([0]) for _ in range(5))
    assert indexing.getitem(torch.randn(2, 2, 2, 2, 2), five, emulate=True) is NotImplemented
