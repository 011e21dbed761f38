"""Index planning for `a[index]`, `a[index] = value` and the gradient of `a[index]` on CUDA tensors.

An index expression is split in two stages (the reference's `IndexPlan`, `genesis/backends/cuda.py:46-75, 1006-1306`):

1. everything basic (ints, slices, `None`, `...`) becomes a strided VIEW of the tensor, no kernel;
2. tensor indices (int32 / int64, any broadcastable shapes; bool masks are compacted to the flat positions of their
   true elements by the block-scan `nonzero` kernels, over the masked dims collapsed into one) are executed by ONE
   kernel (`csrc/indexing.cu`): `out[pre, B, post] = v[pre, idx_0[B], .., idx_k[B], post]`, with the indexed dims
   adjacent (`pre` / `post` around them) or, as numpy and torch define it, the broadcast block first when they are not.

Writes use the same plan (`index_put`, assignment or atomic accumulation); `a[mask] = scalar` with a mask over leading
dims is a single masked-fill kernel with no host read.  Whatever the plan cannot express (more than 4 index tensors,
> 4-D broadcast shapes, ...) returns `NotImplemented` and the caller falls back (counted, see `dispatch.fallbacks`).

All functions take and return raw `torch.Tensor`s.  `emulate=True` runs stage 2 with plain torch indexing on the
planned operands instead of the kernels, which is how the planner is tested on machines without a GPU.
"""
import numpy as np
import torch

from . import native as N

_INT = (torch.int32, torch.int64)


class Plan:
    __slots__ = ("v", "dims", "idx", "bshape", "pre", "post", "copied", "final_shape")

    def __init__(self, v, dims, idx, bshape, pre, post, copied, final_shape=None):
        self.v, self.dims, self.idx, self.bshape, self.pre, self.post, self.copied = v, dims, idx, bshape, pre, post, copied
        # shape the user sees; differs from `out_shape` when the sides of the indexed block were collapsed
        self.final_shape = self.out_shape if final_shape is None else tuple(final_shape)

    @property
    def out_shape(self):
        return tuple([self.v.shape[d] for d in self.pre] + list(self.bshape) + [self.v.shape[d] for d in self.post])


def _contig(t, emulate):
    if t.is_contiguous():
        return t
    if emulate or not t.is_cuda:
        return t.contiguous()
    r = N.contiguous(t)
    return t.contiguous() if r is NotImplemented else r


def _normalise(t, index):
    items = list(index) if isinstance(index, tuple) else [index]
    out = []
    for it in items:
        if isinstance(it, (list, np.ndarray)):
            it = torch.as_tensor(it, device=t.device)
        if isinstance(it, bool):
            return None
        if isinstance(it, torch.Tensor):
            if it.device != t.device:
                it = it.to(t.device)
            if it.dtype not in _INT and it.dtype != torch.bool:
                if it.dtype.is_floating_point or it.dtype.is_complex:
                    raise IndexError("tensors used as indices must be long, int or bool tensors")
                it = it.long()
        elif it is not None and it is not Ellipsis and not isinstance(it, (int, slice, np.integer)):
            return None
        out.append(int(it) if isinstance(it, np.integer) else it)
    return out


def make_plan(t, index, writable=False, emulate=False):
    """Plan for `t[index]`: a `Plan` whose `v` is a view of `t` (stage 1) plus the tensor-index stage, or
    `NotImplemented`.  With `writable`, `v` always aliases `t` (no contiguous copies are taken); a mask over dims that
    cannot be collapsed in place then returns `NotImplemented`."""
    items = _normalise(t, index)
    if items is None:
        return NotImplemented
    consumed = 0
    for it in items:
        if isinstance(it, torch.Tensor):
            consumed += it.dim() if it.dtype == torch.bool else 1
        elif it is not None and it is not Ellipsis:
            consumed += 1
    n_ell = sum(1 for it in items if it is Ellipsis)
    if n_ell > 1 or consumed > t.dim():
        raise IndexError(f"too many indices for tensor of dimension {t.dim()}")
    fill = [slice(None)] * (t.dim() - consumed)
    if n_ell:
        pos = next(i for i, it in enumerate(items) if it is Ellipsis)
        items = items[:pos] + fill + items[pos + 1:]
    else:
        items = items + fill
    # (torch's rule, which differs from numpy's: an integer is applied as a view before adjacency is decided)
    basic, adv, vd = [], [], 0
    for it in items:
        if it is None:
            basic.append(None)
            vd += 1
        elif isinstance(it, int):
            basic.append(it)
        elif isinstance(it, slice):
            basic.append(it)
            vd += 1
        elif it.dtype == torch.bool:
            k = it.dim()
            if k == 0:
                return NotImplemented
            basic.extend([slice(None)] * k)
            adv.append((vd, k, it))
            vd += k
        else:
            basic.append(slice(None))
            adv.append((vd, 1, it))
            vd += 1
    v = t[tuple(basic)] if basic else t
    if not adv:
        return Plan(v, [], [], (), list(range(v.dim())), [], False)
    copied = False
    dims, idx, shift = [], [], 0
    for vd, k, it in adv:
        d = vd - shift
        if it.dtype == torch.bool:
            if tuple(v.shape[d:d + k]) != tuple(it.shape):
                raise IndexError(f"The shape of the mask {list(it.shape)} at index {d} does not match the shape of "
                                 f"the indexed tensor {list(v.shape)} at index {d}")
            if k > 1:
                merged = list(v.shape[:d]) + [int(np.prod(it.shape))] + list(v.shape[d + k:])
                try:
                    v = v.view(merged)
                except RuntimeError:
                    if writable:
                        return NotImplemented
                    v = _contig(v, emulate).view(merged)
                    copied = True
                shift += k - 1
            m = _contig(it, emulate)
            flat = torch.nonzero(m.reshape(-1)).reshape(-1) if (emulate or not m.is_cuda) else N.nonzero_flat(m)
            if flat is NotImplemented:
                return NotImplemented
            idx.append(flat)
        else:
            idx.append(it)
        dims.append(d)
    try:
        bshape = tuple(torch.broadcast_shapes(*[i.shape for i in idx]))
    except RuntimeError as e:
        raise IndexError(f"shape mismatch: indexing tensors could not be broadcast together: {e}") from None
    adjacent = all(b == a + 1 for a, b in zip(dims, dims[1:]))
    if adjacent:
        pre, post = list(range(dims[0])), list(range(dims[-1] + 1, v.dim()))
    else:
        pre, post = [], [d for d in range(v.dim()) if d not in dims]
    if len(idx) > 4 or len(bshape) > 4:
        return NotImplemented
    if len(pre) > 3 or len(post) > 3:
        if not adjacent:
            return NotImplemented
        # collapse each side into one dim (possible in place on contiguous data only)
        final = [v.shape[d] for d in pre] + list(bshape) + [v.shape[d] for d in post]
        mid = [v.shape[d] for d in dims]
        merged = [int(np.prod([v.shape[d] for d in pre]))] + mid + [int(np.prod([v.shape[d] for d in post]))]
        try:
            v = v.view(merged)
        except RuntimeError:
            if writable:
                return NotImplemented
            v = _contig(v, emulate).view(merged)
            copied = True
        dims = list(range(1, 1 + len(mid)))
        pre, post = [0], [1 + len(mid)]
        return Plan(v, dims, idx, bshape, pre, post, copied, final)
    return Plan(v, dims, idx, bshape, pre, post, copied)


def _emulated_get(p):
    order = p.pre + p.dims + p.post
    w = p.v.permute(order)
    key = tuple([slice(None)] * len(p.pre) + [i.long() for i in p.idx])
    return w[key].contiguous()


def _emulated_put(p, val, add):
    order = p.pre + p.dims + p.post
    w = p.v.permute(order)
    key = tuple([slice(None)] * len(p.pre) + [i.long() for i in p.idx])
    if not isinstance(val, torch.Tensor):
        val = torch.full(p.out_shape, val, dtype=p.v.dtype, device=p.v.device)
    val = val.reshape(p.out_shape)
    if not add:
        w[key] = val
        return
    lin = torch.arange(w.numel(), device=w.device).reshape(w.shape)[key].reshape(-1)
    flat = torch.zeros(w.numel(), dtype=w.dtype, device=w.device)
    flat.index_add_(0, lin, val.reshape(-1).to(w.dtype))
    w.add_(flat.reshape(w.shape))


def getitem(t, index, emulate=False):
    """`t[index]` (a view when the index is basic, a new tensor otherwise), or `NotImplemented`."""
    p = make_plan(t, index, emulate=emulate)
    if p is NotImplemented:
        return NotImplemented
    if not p.idx:
        return p.v
    if emulate:
        return _emulated_get(p).reshape(p.final_shape)
    r = N.index_get(p.v, p.dims, p.idx, p.bshape, p.pre, p.post)
    return r if r is NotImplemented else r.reshape(p.final_shape)


def _value_for(p, value, dtype, emulate):
    """`value` shaped for the plan: a python scalar stays one, a tensor becomes contiguous [pre, B, post] of `dtype`."""
    if not isinstance(value, torch.Tensor):
        return value
    if value.numel() == 1 and value.dim() == 0 and not value.is_cuda:
        return value.item()
    if value.device != p.v.device:
        value = value.to(p.v.device)
    if value.dtype != dtype:
        from . import dispatch as K
        value = value.to(dtype) if emulate else K.to_dtype(value, dtype)
    shape = p.final_shape
    if tuple(value.shape) != shape:
        value = value.expand(shape)
    return _contig(value, emulate).reshape(p.out_shape)


def setitem_(t, index, value, emulate=False):
    """`t[index] = value` in place.  Returns `t`, or `NotImplemented` when the plan cannot run natively."""
    from . import dispatch as K
    scalar = not isinstance(value, torch.Tensor) or (value.dim() == 0 and not value.is_cuda)
    # a[mask] = scalar over leading dims: one masked-fill kernel, no host read of the count
    key = index[0] if isinstance(index, tuple) and len(index) == 1 else index
    if scalar and isinstance(key, torch.Tensor) and key.dtype == torch.bool and not emulate and t.is_cuda \
            and t.is_contiguous() and key.is_cuda:
        r = N.masked_fill_(t, _contig(key, False), float(value))
        if r is not NotImplemented:
            return t
    p = make_plan(t, index, writable=True, emulate=emulate)
    if p is NotImplemented:
        return NotImplemented
    val = _value_for(p, value, t.dtype, emulate)
    if not p.idx:
        if p.v.numel() == 0:
            return t
        if isinstance(val, torch.Tensor):
            if emulate:
                p.v.copy_(val)
            else:
                K.copy_(p.v, val)
        elif emulate:
            p.v.fill_(val)
        elif K.fill_view_(p.v, val) is NotImplemented:
            return NotImplemented
        return t
    if emulate:
        _emulated_put(p, val, add=False)
        return t
    r = N.index_put_(p.v, p.dims, p.idx, p.bshape, p.pre, p.post, val, add=False)
    return NotImplemented if r is NotImplemented else t


def getitem_backward(shape, index, g, emulate=False):
    """Gradient of `a[index]` with respect to `a` (shape `shape`): zeros with `g` added at the indexed positions,
    duplicates adding up.  `NotImplemented` when the plan cannot run natively."""
    from . import dispatch as K
    out = torch.empty(shape, dtype=g.dtype, device=g.device)
    if emulate or not out.is_cuda:
        out.zero_()
    else:
        K.zero_(out)
    p = make_plan(out, index, writable=True, emulate=emulate)
    if p is NotImplemented:
        return NotImplemented
    val = _value_for(p, g, out.dtype, emulate)
    if not p.idx:
        # a basic index addresses every element at most once: the sum is an assignment into the zeros
        if p.v.numel():
            if emulate:
                p.v.copy_(val)
            else:
                K.copy_(p.v, val)
        return out
    if emulate:
        _emulated_put(p, val, add=True)
        return out
    r = N.index_put_(p.v, p.dims, p.idx, p.bshape, p.pre, p.post, val, add=True)
    return NotImplemented if r is NotImplemented else out
