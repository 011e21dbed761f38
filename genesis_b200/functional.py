"""Non-differentiable tensor helpers. Parity: reference `genesis/functional.py:12-240`."""
import torch

from .tensor import Tensor
from .ops import dispatch as K


def _r(x):
    return x._t if isinstance(x, Tensor) else x


def _w(t):
    return Tensor._wrap(t)


def triu(a, k=0):
    return _w(K.triu_tril(a._t, k, True))


def tril(a, k=0):
    return _w(K.triu_tril(a._t, k, False))


def isinf(a):
    return _w(torch.isinf(a._t))


def isnan(a):
    return _w(torch.isnan(a._t))


def isfinite(a):
    return _w(torch.isfinite(a._t))


def argsort(a, dim=-1, descending=False):
    return _w(K.sort(a._t, dim, descending)[1])


def sort(a, dim=-1, descending=False):
    v, i = K.sort(a._t, dim, descending)
    return _w(v), _w(i)


def bincount(a, weights=None, minlength=0):
    return _w(K.bincount(a._t, None if weights is None else _r(weights), minlength))


def nonzero(a, as_tuple=False):
    out = K.nonzero(a._t)
    return tuple(_w(out[:, d]) for d in range(out.shape[1])) if as_tuple else _w(out)


def allclose(a, b, rtol=1e-5, atol=1e-8, equal_nan=False):
    # a 0-d bool tensor, as in the reference (`functional.py:191-216`): `if allclose(..)` and `.item()` both work
    return _w(torch.tensor(bool(torch.allclose(a._t.float(), b._t.float().to(a._t.device), rtol=rtol, atol=atol,
                                               equal_nan=equal_nan)), device=a._t.device))


def _cmp(name):
    def f(a, b):
        return _w(K.compare(name, a._t, _r(b)))
    f.__name__ = name
    return f


eq, ne, gt, ge, lt, le = (_cmp(n) for n in ("eq", "ne", "gt", "ge", "lt", "le"))


def empty(*shape, device=None, dtype="float32", requires_grad=False):
    """Uninitialised tensor (the reference also exports this creation helper from `genesis.functional`)."""
    from . import init
    return init.empty(*shape, device=device, dtype=dtype, requires_grad=requires_grad)


def arange(*args, dtype=None, device=None):
    """`arange(end)`, `arange(start, end)` or `arange(start, end, step)`."""
    from . import init
    return init.arange(*args, device=device, dtype=dtype)


def __getattr__(name):
    """The reference's `genesis.functional` star-imports `genesis.nn.functional` (`functional.py:10`): every name of that
    module resolves here too (lazily, because nn.functional imports this module)."""
    from .nn import functional as _nnf
    try:
        return getattr(_nnf, name)
    except AttributeError:
        raise AttributeError(f"module 'genesis.functional' has no attribute {name!r}") from None
