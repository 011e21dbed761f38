"""Binds operators and methods onto `Tensor`. Parity: reference `genesis/api.py:9-161`."""
from .tensor import Tensor


def bind_tensor_methods():
    from .nn import functional as F
    from . import functional as G
    T = Tensor
    T.__add__ = lambda s, o: F.add(s, o)
    T.__radd__ = lambda s, o: F.add(s, o)
    T.__sub__ = lambda s, o: F.sub(s, o)
    T.__rsub__ = lambda s, o: F.sub_scalar(s, o, reverse=True)
    T.__mul__ = lambda s, o: F.mul(s, o)
    T.__rmul__ = lambda s, o: F.mul(s, o)
    T.__truediv__ = lambda s, o: F.truediv(s, o)
    T.__rtruediv__ = lambda s, o: F.divide_scalar(s, o, reverse=True)
    T.__floordiv__ = lambda s, o: F.floordiv(s, o)
    T.__pow__ = lambda s, o: F.pow(s, o)
    T.__rpow__ = lambda s, o: F.pow_scalar(s, o, reverse=True)
    T.__neg__ = lambda s: F.neg(s)
    T.__abs__ = lambda s: F.abs(s)
    T.__matmul__ = lambda s, o: F.matmul(s, o)
    T.__iadd__ = lambda s, o: F.add_inplace(s, o)
    T.__isub__ = lambda s, o: F.sub_inplace(s, o)
    T.__imul__ = lambda s, o: F.mul_inplace(s, o)
    T.__itruediv__ = lambda s, o: F.div_inplace(s, o)

    T.add, T.sub, T.mul, T.div, T.pow = F.add, F.sub, F.mul, F.truediv, F.pow
    T.neg, T.abs, T.exp, T.log, T.sqrt = F.neg, F.abs, F.exp, F.log, F.sqrt
    T.rsqrt = lambda s: F.pow(s, -0.5)
    T.sin, T.cos, T.tanh = F.sin, F.cos, F.tanh
    T.matmul = T.mm = F.matmul

    T.view = lambda s, *shape: F.view(s, *shape)
    T.reshape = lambda s, *shape: F.reshape(s, *shape)
    T.contiguous = lambda s: F.contiguous(s)
    T.flatten = lambda s, start_dim=0, end_dim=None: F.flatten(s, start_dim, end_dim)
    T.permute = lambda s, *dims: F.permute(s, dims if len(dims) > 1 else dims[0])
    T.transpose = lambda s, dim0, dim1: F.transpose(s, dim0, dim1)
    T.T = property(lambda s: F.permute(s, tuple(reversed(range(s.ndim)))))
    T.t = lambda s: F.t(s)
    T.squeeze = lambda s, dim=None: F.squeeze(s, dim)
    T.unsqueeze = lambda s, dim: F.unsqueeze(s, dim)
    T.expand = lambda s, *shape: F.expand(s, *shape)
    T.broadcast_to = lambda s, shape: F.broadcast_to(s, shape)
    T.clamp = lambda s, min=None, max=None: F.clamp(s, min_val=min, max_val=max)
    T.clip = T.clamp

    T.sum = lambda s, dim=None, keepdim=False: F.sum(s, dim, keepdim)
    T.mean = lambda s, dim=None, keepdim=False: F.mean(s, dim, keepdim)
    T.var = lambda s, dim=None, keepdim=False, unbiased=True: F.var(s, dim, keepdim, unbiased)
    T.std = lambda s, dim=None, keepdim=False, unbiased=True: F.std(s, dim, keepdim, unbiased)
    T.max = lambda s, dim=None, keepdim=False: F.max(s, dim, keepdim)
    T.min = lambda s, dim=None, keepdim=False: F.min(s, dim, keepdim)
    T.argmax = lambda s, dim=None, keepdim=False: F.argmax(s, dim, keepdim)
    T.argmin = lambda s, dim=None, keepdim=False: F.argmin(s, dim, keepdim)
    T.argsort = lambda s, dim=-1, descending=False: G.argsort(s, dim, descending)
    T.nonzero = lambda s, as_tuple=False: G.nonzero(s, as_tuple)
    T.topk = lambda s, k, dim=-1, largest=True, sorted=True: F.topk(s, k, dim, largest, sorted)

    T.eq, T.ne, T.lt, T.le, T.gt, T.ge = G.eq, G.ne, G.lt, G.le, G.gt, G.ge
    T.__eq__, T.__ne__, T.__lt__, T.__le__, T.__gt__, T.__ge__ = G.eq, G.ne, G.lt, G.le, G.gt, G.ge
    T.__hash__ = lambda s: id(s)
    T.__invert__ = lambda s: Tensor._wrap(~s._t)
    T.__and__ = lambda s, o: Tensor._wrap(s._t & (o._t if isinstance(o, Tensor) else o))
    T.__or__ = lambda s, o: Tensor._wrap(s._t | (o._t if isinstance(o, Tensor) else o))

    T.long = lambda s: s.to_dtype("int64")
    T.int = lambda s: s.to_dtype("int32")
    T.float = lambda s: s.to_dtype("float32")
    T.double = lambda s: s.to_dtype("float64")
    T.half = lambda s: s.to_dtype("float16")
    T.bfloat16 = lambda s: s.to_dtype("bfloat16")
    T.bool = lambda s: s.to_dtype("bool")
    T.isinf, T.isnan, T.isfinite = G.isinf, G.isnan, G.isfinite


def bind_nn_functional_methods():
    from .nn import functional as F
    T = Tensor
    T.relu = F.relu
    T.sigmoid = F.sigmoid
    T.softmax = lambda s, dim=-1: F.softmax(s, dim)
    T.log_softmax = lambda s, dim=-1: F.log_softmax(s, dim)
    T.repeat_interleave = lambda s, repeats, dim=None: F.repeat_interleave(s, repeats, dim)
    T.scatter_add = lambda s, dim, index, src: F.scatter_add(s, dim, index, src)
    T.dropout = lambda s, p=0.5, training=True: F.dropout(s, p, training)
    T.__getitem__ = lambda s, key: F.getitem(s, key)
    T.__setitem__ = lambda s, key, value: F.setitem(s, key, value)
    T.__len__ = lambda s: s.shape[0] if s.shape else 0
    T.gather = lambda s, dim, index: F.gather(s, dim, index)
    T.scatter = lambda s, dim, index, src: F.scatter(s, dim, index, src)

    def scatter_(s, dim, index, src):
        from .ops import dispatch as K
        K.scatter_(s._t, dim, index._t, src._t if isinstance(src, Tensor) else src)
        s._version += 1
        return s
    T.scatter_ = scatter_
    T.masked_fill = lambda s, mask, value: F.where(mask, value, s)
    T.split = lambda s, dim=0, split_size_or_sections=1: F.split(s, dim, split_size_or_sections)
