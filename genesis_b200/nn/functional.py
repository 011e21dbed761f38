"""Differentiable operations (`Function` subclasses) and their functional wrappers.

Parity: reference `genesis/nn/functional.py` (op list, argument names such as
`sum(a, axis, keepdims)`, AMP policy per op — the reference's policy
table: matmul/relu/gelu/attention run in the autocast dtype; pow/log/exp/sqrt/
sum/mean/logsumexp/sigmoid/tanh/softmax/layer-norm run in float32; shape, index
and scalar ops preserve dtypes) plus the fused ops the reference builds from
Triton kernels (`nn/triton_ops/*`, `nn/attention.py`, `nn/layer_norm.py`).
All functions here are `raw`: forward/backward work on torch tensors and call
`genesis_b200.ops.dispatch`.
"""
import builtins
import math

import torch

from ..function import Function, AMPPolicy, cast
from ..tensor import Tensor
from ..ops import dispatch as K
from ..amp_state import amp_state, shadow_of, stacked_shadow_of
from .. import random as _random

_pysum, _pymax, _pymin, _pyabs, _pypow = builtins.sum, builtins.max, builtins.min, builtins.abs, builtins.pow


def _is_t(x):
    return isinstance(x, Tensor)


def _as_tensor_like(x, ref):
    """Python scalar / numpy -> Tensor on ref's device."""
    if isinstance(x, Tensor):
        return x
    return Tensor._wrap(torch.as_tensor(x, device=ref._t.device))


# ================================ elementwise binary ===============================
class _Binary(Function):
    raw = True
    op = None

    @classmethod
    def forward(cls, ctx, a, b):
        ctx.shapes = (a.shape, b.shape)
        cls._save(ctx, a, b)
        return cls._fwd(a, b)


class EWiseAdd(_Binary):
    _save = staticmethod(lambda ctx, a, b: None)
    _fwd = staticmethod(K.add)

    @staticmethod
    def backward(ctx, g):
        sa, sb = ctx.shapes
        na, nb = ctx.needs_input_grad
        return (K.sum_to_shape(g, sa) if na else None, K.sum_to_shape(g, sb) if nb else None)


class EWiseSub(_Binary):
    _save = staticmethod(lambda ctx, a, b: None)
    _fwd = staticmethod(K.sub)

    @staticmethod
    def backward(ctx, g):
        sa, sb = ctx.shapes
        na, nb = ctx.needs_input_grad
        return (K.sum_to_shape(g, sa) if na else None,
                K.sum_to_shape(K.unary("neg", g), sb) if nb else None)


class EWiseMul(_Binary):
    _save = staticmethod(lambda ctx, a, b: ctx.save_for_backward(a, b))
    _fwd = staticmethod(K.mul)

    @staticmethod
    def backward(ctx, g):
        a, b = ctx.saved_tensors
        na, nb = ctx.needs_input_grad
        return (K.sum_to_shape(K.mul(g, b), a.shape) if na else None,
                K.sum_to_shape(K.mul(g, a), b.shape) if nb else None)


class EWiseDiv(_Binary):
    _save = staticmethod(lambda ctx, a, b: ctx.save_for_backward(a, b))
    _fwd = staticmethod(K.div)

    @staticmethod
    def backward(ctx, g):
        a, b = ctx.saved_tensors
        na, nb = ctx.needs_input_grad
        ga = K.sum_to_shape(K.div(g, b), a.shape) if na else None
        gb = None
        if nb:
            gb = K.unary("neg", K.div(K.mul(g, a), K.mul(b, b)))
            gb = K.sum_to_shape(gb, b.shape)
        return ga, gb


class Maximum(_Binary):
    _save = staticmethod(lambda ctx, a, b: ctx.save_for_backward(a, b))
    _fwd = staticmethod(K.maximum)

    @staticmethod
    def backward(ctx, g):
        a, b = ctx.saved_tensors
        m = K.compare("ge", a, b)
        ga = K.sum_to_shape(K.mul(g, m.to(g.dtype)), a.shape)
        gb = K.sum_to_shape(K.mul(g, (~m).to(g.dtype)), b.shape)
        return ga, gb


# ================================== scalar ops ====================================
class AddScalar(Function):
    raw = True
    amp_policy = AMPPolicy.PRESERVE

    @staticmethod
    def forward(ctx, a, s):
        return K.add(a, s)

    @staticmethod
    def backward(ctx, g):
        return g


class SubScalar(Function):
    raw = True
    amp_policy = AMPPolicy.PRESERVE

    @staticmethod
    def forward(ctx, a, s, reverse=False):
        ctx.reverse = reverse
        return K.sub(s, a) if reverse else K.sub(a, s)

    @staticmethod
    def backward(ctx, g):
        return K.unary("neg", g) if ctx.reverse else g


class MulScalar(Function):
    raw = True
    amp_policy = AMPPolicy.PRESERVE

    @staticmethod
    def forward(ctx, a, s):
        ctx.s = s
        return K.mul(a, s)

    @staticmethod
    def backward(ctx, g):
        return K.mul(g, ctx.s)


class DivScalar(Function):
    raw = True
    amp_policy = AMPPolicy.PRESERVE

    @staticmethod
    def forward(ctx, a, s, reverse=False):
        ctx.s, ctx.reverse = s, reverse
        if reverse:
            ctx.save_for_backward(a)
            return K.div(s, a)
        return K.div(a, s)

    @staticmethod
    def backward(ctx, g):
        if ctx.reverse:
            (a,) = ctx.saved_tensors
            return K.unary("neg", K.div(K.mul(g, ctx.s), K.mul(a, a)))
        return K.div(g, ctx.s)


class PowScalar(Function):
    raw = True
    amp_policy = AMPPolicy.FP32

    @staticmethod
    def forward(ctx, a, s, reverse=False):
        ctx.s, ctx.reverse = s, reverse
        out = K.rpow_scalar(a, s) if reverse else K.pow_scalar(a, s)
        ctx.save_for_backward(out if reverse else a)
        return out

    @staticmethod
    def backward(ctx, g):
        (t,) = ctx.saved_tensors
        if ctx.reverse:      # d/dx s**x = s**x * ln s
            return K.mul(g, K.mul(t, math.log(ctx.s)))
        return K.mul(g, K.mul(K.pow_scalar(t, ctx.s - 1), ctx.s))


class PowTensor(Function):
    """tensor ** tensor (the reference leaves this unimplemented, `functional.py:534-542`)."""
    raw = True
    amp_policy = AMPPolicy.FP32

    @staticmethod
    def forward(ctx, a, b):
        out = torch.pow(a, b)
        ctx.save_for_backward(a, b, out)
        return out

    @staticmethod
    def backward(ctx, g):
        a, b, out = ctx.saved_tensors
        ga = K.sum_to_shape(g * b * torch.pow(a, b - 1), a.shape)
        gb = K.sum_to_shape(g * out * torch.log(a), b.shape)
        return ga, gb


# ==================================== unary =======================================
def _make_unary(name, policy, save):
    class _U(Function):
        raw = True
        amp_policy = policy

        @staticmethod
        def forward(ctx, a):
            y = K.unary(name, a)
            if save == "y":
                ctx.save_for_backward(None, y)
            elif save == "x":
                ctx.save_for_backward(a, None)
            return y

        @staticmethod
        def backward(ctx, g):
            if save is None:
                return K.unary_bwd(name, g, None, None)
            x, y = ctx.saved_tensors
            return K.unary_bwd(name, g, x, y)
    _U.__name__ = _U.__qualname__ = name.capitalize()
    return _U


Negate = _make_unary("neg", AMPPolicy.PRESERVE, None)
Sin = _make_unary("sin", AMPPolicy.FP32, "x")
Cos = _make_unary("cos", AMPPolicy.FP32, "x")
Log = _make_unary("log", AMPPolicy.FP32, "x")
Exp = _make_unary("exp", AMPPolicy.FP32, "y")
Sqrt = _make_unary("sqrt", AMPPolicy.FP32, "y")
Abs = _make_unary("abs", AMPPolicy.PRESERVE, "x")
Sigmoid = _make_unary("sigmoid", AMPPolicy.FP32, "y")
Tanh = _make_unary("tanh", AMPPolicy.FP32, "y")
ReLU = _make_unary("relu", AMPPolicy.FP16, "x")
SiLUFunction = _make_unary("silu", AMPPolicy.PRESERVE, "x")
GELUFunction = _make_unary("gelu", AMPPolicy.FP16, "x")


class Clamp(Function):
    raw = True
    amp_policy = AMPPolicy.PRESERVE

    @staticmethod
    def forward(ctx, a, lo, hi):
        ctx.save_for_backward(a)
        ctx.lo, ctx.hi = lo, hi
        return K.clamp(a, lo, hi)

    @staticmethod
    def backward(ctx, g):
        (a,) = ctx.saved_tensors
        m = torch.ones_like(a, dtype=torch.bool)
        if ctx.lo is not None:
            m &= K.compare("ge", a, ctx.lo)
        if ctx.hi is not None:
            m &= K.compare("le", a, ctx.hi)
        return K.mul(g, m.to(g.dtype))


class Where(Function):
    raw = True
    amp_policy = AMPPolicy.PRESERVE

    @staticmethod
    def forward(ctx, cond, x, y):
        ctx.save_for_backward(cond)
        ctx.shapes = (x.shape if isinstance(x, torch.Tensor) else None,
                      y.shape if isinstance(y, torch.Tensor) else None)
        return K.where(cond, x, y)

    @staticmethod
    def backward(ctx, g):
        (cond,) = ctx.saved_tensors
        sx, sy = ctx.shapes
        grads = [None]
        zero = 0.0
        if sx is not None:
            grads.append(K.sum_to_shape(K.where(cond, g, zero), sx))
        if sy is not None:
            grads.append(K.sum_to_shape(K.where(cond, zero, g), sy))
        return tuple(grads)


class Clone(Function):
    raw = True
    amp_policy = AMPPolicy.PRESERVE

    @staticmethod
    def forward(ctx, a):
        return K.clone(a)

    @staticmethod
    def backward(ctx, g):
        return g


class ToDevice(Function):
    raw = True
    amp_policy = AMPPolicy.PRESERVE

    @staticmethod
    def forward(ctx, a, device):
        ctx.src = a.device
        return a.to(device)

    @staticmethod
    def backward(ctx, g):
        return g.to(ctx.src)


# ================================== reductions ====================================
def _axes(axis):
    if axis is None:
        return None
    if isinstance(axis, int):
        return (axis,)
    return tuple(axis)


def _expand_reduced(g, in_shape, axes, keepdims):
    """Reshape a reduced gradient so it broadcasts against the input shape."""
    if axes is None:
        return g.reshape((1,) * len(in_shape))
    if keepdims:
        return g
    shape = list(in_shape)
    for a in axes:
        shape[a % len(in_shape)] = 1
    return g.reshape(shape)


class Summation(Function):
    raw = True
    amp_policy = AMPPolicy.FP32

    @staticmethod
    def forward(ctx, a, axis=None, keepdims=False):
        ctx.meta = (a.shape, _axes(axis), keepdims)
        return K.reduce("sum", a, _axes(axis), keepdims)

    @staticmethod
    def backward(ctx, g):
        shape, axes, keep = ctx.meta
        return _expand_reduced(g, shape, axes, keep).expand(shape)


class Mean(Function):
    raw = True
    amp_policy = AMPPolicy.FP32

    @staticmethod
    def forward(ctx, a, axis=None, keepdims=False):
        ctx.meta = (a.shape, _axes(axis), keepdims)
        return K.reduce("mean", a, _axes(axis), keepdims)

    @staticmethod
    def backward(ctx, g):
        shape, axes, keep = ctx.meta
        n = 1
        if axes is None:
            for s in shape:
                n *= s
        else:
            for a in axes:
                n *= shape[a % len(shape)]
        return K.mul(_expand_reduced(g, shape, axes, keep), 1.0 / _pymax(n, 1)).expand(shape)


class _MinMax(Function):
    raw = True
    amp_policy = AMPPolicy.PRESERVE
    name = "max"

    @classmethod
    def forward(cls, ctx, a, axis=None, keepdims=False):
        out = K.reduce(cls.name, a, _axes(axis), keepdims)
        ctx.save_for_backward(a, out)
        ctx.meta = (_axes(axis), keepdims)
        return out

    @staticmethod
    def backward(ctx, g):
        a, out = ctx.saved_tensors
        axes, keep = ctx.meta
        o = _expand_reduced(out, a.shape, axes, keep)
        mask = K.compare("eq", a, o.expand(a.shape)).to(g.dtype)
        cnt = K.reduce("sum", mask, axes, True) if axes is not None else K.reduce("sum", mask).reshape((1,) * a.dim())
        gg = _expand_reduced(g, a.shape, axes, keep)
        return K.div(K.mul(mask, gg.expand(a.shape)), cnt.expand(a.shape))


class Max(_MinMax):
    name = "max"


class Min(_MinMax):
    name = "min"


class LogSumExp(Function):
    raw = True
    amp_policy = AMPPolicy.FP32

    @staticmethod
    def forward(ctx, a, axis=None):
        axes = _axes(axis)
        m = K.reduce("max", a, axes, True) if axes is not None else K.reduce("max", a).reshape((1,) * a.dim())
        e = K.unary("exp", K.sub(a, m.expand(a.shape)))
        s = K.reduce("sum", e, axes, True) if axes is not None else K.reduce("sum", e).reshape((1,) * a.dim())
        out = K.add(K.unary("log", s), m)
        ctx.save_for_backward(a, out)
        ctx.axes = axes
        if axes is None:
            return out.reshape(())
        return out.reshape([s_ for i, s_ in enumerate(a.shape) if i not in {x % a.dim() for x in axes}])

    @staticmethod
    def backward(ctx, g):
        a, out = ctx.saved_tensors
        p = K.unary("exp", K.sub(a, out.expand(a.shape)))
        return K.mul(p, g.reshape(out.shape).expand(a.shape))


# ==================================== matmul ======================================
class Matmul(Function):
    raw = True
    amp_policy = AMPPolicy.FP16

    @staticmethod
    def forward(ctx, a, b):
        ctx.save_for_backward(a, b)
        return K.matmul(a, b)

    @staticmethod
    def backward(ctx, g):
        a, b = ctx.saved_tensors
        na, nb = ctx.needs_input_grad
        ga = gb = None
        a1, b1 = a.dim() == 1, b.dim() == 1
        aa = a.unsqueeze(0) if a1 else a
        bb = b.unsqueeze(-1) if b1 else b
        gg = g
        if a1:
            gg = gg.unsqueeze(-2)
        if b1:
            gg = gg.unsqueeze(-1)
        if na:
            ga = K.matmul(gg, bb.transpose(-1, -2))
            ga = K.sum_to_shape(ga, aa.shape) if ga.shape != aa.shape else ga
            if a1:
                ga = ga.reshape(a.shape)
        if nb:
            gb = K.matmul(aa.transpose(-1, -2), gg)
            gb = K.sum_to_shape(gb, bb.shape) if gb.shape != bb.shape else gb
            if b1:
                gb = gb.reshape(b.shape)
        return ga, gb


class LinearFunction(Function):
    """y = x @ W^T + b as one node. Under autocast the float32 master weight is cast once
    per region (cached) and the weight gradient is produced directly in float32 by the
    GEMM epilogue, so no low-precision dW round trip exists."""
    raw = True
    amp_policy = AMPPolicy.PRESERVE

    @staticmethod
    def forward(ctx, x, w, b, compute_dtype):
        wd = w.dtype
        if compute_dtype is not None:
            if x.dtype != compute_dtype:
                x = K.to_dtype(x, compute_dtype)
            wc = _cached_param_cast(w, compute_dtype)
        else:
            wc = w
            if x.dtype != w.dtype:
                x = K.to_dtype(x, w.dtype)
        ctx.save_for_backward(x, wc)
        ctx.meta = (wd, None if b is None else b.dtype)
        return K.linear(x, wc, b)

    @staticmethod
    def backward(ctx, g):
        x, wc = ctx.saved_tensors
        wd, bd = ctx.meta
        need = ctx.needs_input_grad
        if g.dtype != x.dtype:
            g = K.to_dtype(g, x.dtype)
        if not g.is_contiguous():
            g = K.contiguous(g)
        gx = K.linear_dgrad(g, wc) if need[0] else None
        gw = None
        if need[1]:
            slot = _grad_slot(ctx, 1, wd, wc.shape)
            if slot is None:
                gw = K.linear_wgrad(g, x, out_dtype=wd)
            else:
                # the weight is a leaf with a preallocated gradient slot (a DDP bucket view): the GEMM writes or
                # accumulates there, and the engine recognises the slot instead of copying into it
                buf, accumulate = slot
                gw = K.linear_wgrad(g, x, out_dtype=buf.dtype, accum=buf if accumulate else None,
                                    out=None if accumulate else buf)
        gb = None
        if bd is not None and len(need) > 2 and need[2]:
            gb = K.bias_grad(g, bd)
        return (gx, gw, gb) if bd is not None else (gx, gw)


def _grad_slot(ctx, i, dtype, shape):
    """(slot, accumulate) when input `i` of the node is a leaf whose gradient has a preallocated home
    (`Tensor._grad_buf`, set by DistributedDataParallel) that a kernel may target directly: `accumulate` is False
    when the leaf has no gradient yet (the kernel overwrites the slot) and True when its gradient already lives in
    the slot (the kernel adds to it).  None in every other case (hooks, foreign gradient tensor, dtype mismatch)."""
    edges = getattr(ctx, "edges", None)
    if not edges or i >= len(edges) or edges[i] is None:
        return None
    leaf = edges[i].leaf
    if leaf is None or leaf._grad_buf is None or leaf._hooks:
        return None
    buf = leaf._grad_buf
    # (the slot may be narrower than the parameter: DDP's 16-bit wire format; the GEMM then writes that dtype)
    if not buf.dtype.is_floating_point or not buf.is_contiguous() or tuple(buf.shape) != tuple(shape):
        return None
    if leaf.grad is None:
        return buf, False
    if leaf.grad._t.data_ptr() == buf.data_ptr():
        return buf, True
    return None


def _stacked_grad_slot(ctx, first, sizes, dtype, cols):
    """One [sum(sizes), cols] view over the gradient slots of inputs first .. first + len(sizes) - 1 when each has a
    slot (`_grad_slot`), all in the same state, lying back to back in memory in that order; (None, False) otherwise."""
    slots = []
    for j, n in enumerate(sizes):
        sl = _grad_slot(ctx, first + j, dtype, (n, cols))
        if sl is None or (slots and sl[1] != slots[0][1]):
            return None, False
        slots.append(sl)
    es = slots[0][0].element_size()
    if len({sl[0].dtype for sl in slots}) != 1:
        return None, False
    dtype = slots[0][0].dtype
    for (a, _), (b, _) in zip(slots, slots[1:]):
        if a.data_ptr() + a.numel() * es != b.data_ptr() or a.untyped_storage().data_ptr() != b.untyped_storage().data_ptr():
            return None, False
    head = slots[0][0]
    stacked = torch.empty(0, dtype=dtype, device=head.device).set_(
        head.untyped_storage(), head.storage_offset(), (builtins.sum(sizes), cols), (cols, 1))
    return stacked, slots[0][1]


def _cached_param_cast(w, dtype):
    if w.dtype == dtype:
        return w
    lp = shadow_of(w, dtype)                      # a copy the optimizer keeps current: no conversion kernel
    if lp is not None:
        return lp
    key = ("raw", w.data_ptr(), w._version, dtype)
    hit = amp_state.cache.get(key)
    if hit is not None and hit[0] is w:
        return hit[1]
    wc = K.to_dtype(w, dtype)
    if amp_state.enabled:
        amp_state.cache[key] = (w, wc)
    return wc


def linear(x, weight, bias=None):
    cd = amp_state.dtype if amp_state.enabled else None
    if bias is None:
        return LinearFunction.apply(x, weight, None, cd)
    return LinearFunction.apply(x, weight, bias, cd)


# ================================ shape / view ops ================================
class _ViewOp(Function):
    raw = True
    amp_policy = AMPPolicy.PRESERVE


class Reshape(_ViewOp):
    @staticmethod
    def forward(ctx, a, shape):
        ctx.shape = a.shape
        return a.reshape(shape)

    @staticmethod
    def backward(ctx, g):
        return g.reshape(ctx.shape)


class Permute(_ViewOp):
    @staticmethod
    def forward(ctx, a, dims):
        ctx.dims = dims
        return a.permute(dims)

    @staticmethod
    def backward(ctx, g):
        inv = [0] * len(ctx.dims)
        for i, d in enumerate(ctx.dims):
            inv[d % len(inv)] = i
        return g.permute(inv)


class Transpose(_ViewOp):
    @staticmethod
    def forward(ctx, a, d0, d1):
        ctx.d = (d0, d1)
        return a.transpose(d0, d1)

    @staticmethod
    def backward(ctx, g):
        return g.transpose(*ctx.d)


class Contiguous(_ViewOp):
    @staticmethod
    def forward(ctx, a):
        return K.contiguous(a)

    @staticmethod
    def backward(ctx, g):
        return g


class Expand(_ViewOp):
    @staticmethod
    def forward(ctx, a, shape):
        ctx.shape = a.shape
        return a.expand(shape)

    @staticmethod
    def backward(ctx, g):
        return K.sum_to_shape(g, ctx.shape)


class BroadcastTo(Expand):
    pass


class Squeeze(_ViewOp):
    @staticmethod
    def forward(ctx, a, dim):
        ctx.shape = a.shape
        return a.squeeze() if dim is None else a.squeeze(dim)

    @staticmethod
    def backward(ctx, g):
        return g.reshape(ctx.shape)


class Unsqueeze(_ViewOp):
    @staticmethod
    def forward(ctx, a, dim):
        ctx.shape = a.shape
        return a.unsqueeze(dim)

    @staticmethod
    def backward(ctx, g):
        return g.reshape(ctx.shape)


class Flatten(_ViewOp):
    @staticmethod
    def forward(ctx, a, start, end):
        ctx.shape = a.shape
        return a.flatten(start, end)

    @staticmethod
    def backward(ctx, g):
        return g.reshape(ctx.shape)


class Stack(_ViewOp):
    @staticmethod
    def forward(ctx, tensors, dim):
        ctx.dim = dim
        return K.stack(list(tensors), dim)

    @staticmethod
    def backward(ctx, g):
        return tuple(K.contiguous(x) for x in g.unbind(ctx.dim))


class Cat(_ViewOp):
    @staticmethod
    def forward(ctx, tensors, dim):
        ctx.dim = dim
        ctx.sizes = [t.shape[dim] for t in tensors]
        return K.cat(list(tensors), dim)

    @staticmethod
    def backward(ctx, g):
        return tuple(g.split(ctx.sizes, ctx.dim))


class Split(_ViewOp):
    @staticmethod
    def forward(ctx, a, sizes, dim):
        pieces = a.split(sizes, dim)
        ctx.meta = (dim, a.shape, [p.shape[dim] for p in pieces])
        return tuple(pieces)

    @staticmethod
    def backward(ctx, *gs):
        dim, shape, sizes = ctx.meta
        ref = next(x for x in gs if x is not None)
        if all(x is not None for x in gs):
            return K.cat(list(gs), dim)
        out = K.zeros(shape, ref.dtype, ref.device)
        for gpart, piece in zip(gs, out.split(sizes, dim)):
            if gpart is not None:
                K.copy_(piece, gpart)
        return out


# ==================================== indexing =====================================
def _raw_index(index):
    """Convert Tensors inside an index expression to torch tensors."""
    if isinstance(index, Tensor):
        t = index._t
        return t if t.dtype in (torch.bool, torch.int64, torch.int32) else t.long()
    if isinstance(index, tuple):
        return tuple(_raw_index(i) for i in index)
    if isinstance(index, list):
        if index and any(isinstance(i, (Tensor, slice, list)) for i in index):
            return tuple(_raw_index(i) for i in index)
        return index
    return index


class GetItem(_ViewOp):
    @staticmethod
    def forward(ctx, a, index):
        ctx.index = index
        ctx.shape = a.shape
        return K.getitem(a, index)

    @staticmethod
    def backward(ctx, g):
        return K.getitem_backward(ctx.shape, ctx.index, g)


def _int_index(t):
    """int32 / int64 index tensors are used as they are (the kernels read both); anything else becomes int64."""
    return t if t.dtype in (torch.int32, torch.int64) else t.long()


class SetItem(_ViewOp):
    """Out-of-place `a[index] = value` for graph purposes; the public `setitem` mutates in place."""

    @staticmethod
    def forward(ctx, a, value, index):
        ctx.index = index
        ctx.vshape = value.shape if isinstance(value, torch.Tensor) else None
        out = K.clone(a)
        K.setitem_(out, index, value)
        return out

    @staticmethod
    def backward(ctx, g):
        ga = K.clone(g)
        K.setitem_(ga, ctx.index, 0)
        if ctx.vshape is None:
            return (ga,)
        gv = K.getitem(g, ctx.index)
        return ga, K.sum_to_shape(gv, ctx.vshape)


class Gather(_ViewOp):
    @staticmethod
    def forward(ctx, a, dim, index):
        ctx.save_for_backward(index)
        ctx.meta = (dim, a.shape)
        return K.gather(a, dim, index)

    @staticmethod
    def backward(ctx, g):
        (index,) = ctx.saved_tensors
        dim, shape = ctx.meta
        return K.scatter_add_into_zeros(shape, dim, index, g)


class Scatter(_ViewOp):
    @staticmethod
    def forward(ctx, a, dim, index, src):
        ctx.save_for_backward(index)
        ctx.dim = dim
        ctx.src_is_tensor = isinstance(src, torch.Tensor)
        return K.scatter(a, dim, index, src)

    @staticmethod
    def backward(ctx, g):
        (index,) = ctx.saved_tensors
        ga = K.scatter(g, ctx.dim, index, 0)
        if ctx.src_is_tensor:
            return ga, None, K.gather(g, ctx.dim, index)
        return (ga,)


class ScatterAddFunction(_ViewOp):
    @staticmethod
    def forward(ctx, a, dim, index, src):
        ctx.save_for_backward(index)
        ctx.dim = dim
        return K.scatter(a, dim, index, src, add=True)

    @staticmethod
    def backward(ctx, g):
        (index,) = ctx.saved_tensors
        return g, None, K.gather(g, ctx.dim, index)


class TopKFunction(_ViewOp):
    @staticmethod
    def forward(ctx, a, k, dim, largest, sorted_):
        vals, idx = K.topk(a, k, dim, largest)
        ctx.save_for_backward(idx)
        ctx.meta = (dim, a.shape)
        return vals, idx

    @staticmethod
    def backward(ctx, gv, gi=None):
        (idx,) = ctx.saved_tensors
        dim, shape = ctx.meta
        return K.scatter_add_into_zeros(shape, dim, idx, gv)


class RepeatInterleaveFunction(_ViewOp):
    @staticmethod
    def forward(ctx, a, repeats, dim):
        ctx.meta = (a.shape, repeats, dim)
        return K.repeat_interleave(a, repeats, dim)

    @staticmethod
    def backward(ctx, g):
        shape, r, dim = ctx.meta
        if dim is None:
            return g.reshape(-1, r).sum(1).reshape(shape)
        d = dim % len(shape)
        new = list(shape[:d]) + [shape[d], r] + list(shape[d + 1:])
        return K.reduce("sum", g.reshape(new), (d + 1,), False)


class EmbeddingFunction(Function):
    """weight[idx] with an accumulating backward (duplicate tokens add up; the reference's
    CUDA scatter keeps only the last write, `functional.py:1383-1386`)."""
    raw = True
    amp_policy = AMPPolicy.PRESERVE

    @staticmethod
    def forward(ctx, weight, idx, compute_dtype=None):
        ctx.save_for_backward(idx)
        ctx.meta = (weight.shape[0], weight.dtype)
        # under autocast the rows come from the cached low-precision copy of the table (shared with a
        # tied lm_head), so the residual stream of the model runs in the autocast dtype
        w = _cached_param_cast(weight, compute_dtype) if compute_dtype is not None else weight
        return K.embedding_fwd(w, idx)

    @staticmethod
    def backward(ctx, g):
        (idx,) = ctx.saved_tensors
        n, dt = ctx.meta
        # handed to the leaf as (indices, rows): scattered straight into an existing gradient when there is one
        from ..tensor import RowScatterGrad
        return RowScatterGrad(g, idx, n, dt)


# ============================== softmax / losses ==================================
class SoftmaxFunction(Function):
    raw = True
    amp_policy = AMPPolicy.FP32

    @staticmethod
    def forward(ctx, x, dim, log):
        y = K.softmax_fwd(x, dim, log)
        ctx.save_for_backward(y)
        ctx.meta = (dim, log)
        return y

    @staticmethod
    def backward(ctx, g):
        (y,) = ctx.saved_tensors
        dim, log = ctx.meta
        return K.softmax_bwd(g, y, dim, log)


class CrossEntropyFunction(Function):
    """Fused softmax cross-entropy over [N, C] logits with integer targets.

    Forward keeps only the logits and one log-sum-exp per row; backward writes
    (softmax - onehot) * grad in one pass (in place over the logits when they are a
    temporary of the graph).  Replaces the reference's log_softmax + one_hot + mul + sum
    chain (`nn/modules/loss.py:77-100`), which materialises several [N, C] float32 arrays.
    """
    raw = True
    amp_policy = AMPPolicy.PRESERVE

    @staticmethod
    def forward(ctx, logits, target, weight, ignore_index, reduction, inplace_backward):
        N = logits.shape[0]
        loss_rows, lse = K.cross_entropy_fwd(logits, target, ignore_index)
        valid = target != ignore_index
        if weight is not None:
            safe_t = torch.where(valid, target, torch.zeros_like(target)).long()
            w_rows = weight.float()[safe_t] * valid.float()
            loss_rows = loss_rows * w_rows
        else:
            w_rows = None
        if reduction == "mean":
            # mean over the rows that are not ignored (reference `nn/modules/loss.py:95-100`)
            denom = valid.sum().float().clamp_min(1.0)
            out = loss_rows.sum() / denom
        elif reduction == "sum":
            denom = None
            out = loss_rows.sum()
        else:
            denom = None
            out = loss_rows
        ctx.save_for_backward(logits, target, lse, w_rows, denom)
        ctx.meta = (ignore_index, reduction, inplace_backward)
        return out

    @staticmethod
    def backward(ctx, g):
        logits, target, lse, w_rows, denom = ctx.saved_tensors
        ignore_index, reduction, inplace = ctx.meta
        N = logits.shape[0]
        g = g.float()
        if reduction == "none":
            rows = g.reshape(-1)
        else:
            rows = g.reshape(()).expand(N)
            if reduction == "mean":
                rows = rows / denom
        if w_rows is not None:
            rows = rows * w_rows
        rows = rows.contiguous()
        return K.cross_entropy_bwd(logits, target, lse, rows, ignore_index, inplace)


# ============================= fused transformer ops ==============================
class FusedRMSNormFunction(Function):
    raw = True
    amp_policy = AMPPolicy.PRESERVE

    @staticmethod
    def forward(ctx, x, w, eps):
        y, rstd = K.rmsnorm_fwd(x, w, eps)
        ctx.save_for_backward(x, w, rstd)
        return y

    @staticmethod
    def backward(ctx, g):
        x, w, rstd = ctx.saved_tensors
        if g.dtype != x.dtype:
            g = K.to_dtype(g, x.dtype)
        dx, dw = K.rmsnorm_bwd(g if g.is_contiguous() else K.contiguous(g), x, w, rstd)
        return dx, (dw if dw.dtype == w.dtype else dw.to(w.dtype))


class AddRMSNormFunction(Function):
    """(s, y) = (x + res, rmsnorm(x + res) * w): the residual addition of a pre-norm block and the normalisation
    that follows it, one kernel forward and one backward (which also folds in the gradient arriving at s along the
    residual path, so backward has no separate gradient additions either)."""
    raw = True
    amp_policy = AMPPolicy.PRESERVE

    @staticmethod
    def forward(ctx, x, res, w, eps):
        if res.dtype != x.dtype:
            res = K.to_dtype(res, x.dtype)
        x = x if x.is_contiguous() else K.contiguous(x)
        res = res if res.is_contiguous() else K.contiguous(res)
        s, y, rstd = K.add_rmsnorm_fwd(x, res, w, eps)
        ctx.save_for_backward(s, w, rstd)
        return s, y

    @staticmethod
    def backward(ctx, gs, gy):
        s, w, rstd = ctx.saved_tensors
        if gy is None:                                   # the normalised output was not used
            return gs, gs, None
        if gy.dtype != s.dtype:
            gy = K.to_dtype(gy, s.dtype)
        gy = gy if gy.is_contiguous() else K.contiguous(gy)
        if gs is None:
            dx, dw = K.rmsnorm_bwd(gy, s, w, rstd)
        else:
            if gs.dtype != s.dtype:
                gs = K.to_dtype(gs, s.dtype)
            gs = gs if gs.is_contiguous() else K.contiguous(gs)
            dx, dw = K.add_rmsnorm_bwd(gy, gs, s, w, rstd)
        return dx, dx, (dw if dw.dtype == w.dtype else dw.to(w.dtype))


def add_rms_norm(x, residual, weight, eps=1e-6):
    """(x + residual, rms_norm(x + residual, weight)) from one fused kernel."""
    return AddRMSNormFunction.apply(x, residual, weight, eps)


class FusedLayerNormFunction(Function):
    raw = True
    amp_policy = AMPPolicy.FP32

    @staticmethod
    def forward(ctx, x, w, b, eps):
        y, mean, rstd = K.layernorm_fwd(x, w, b, eps)
        ctx.save_for_backward(x, w, mean, rstd)
        ctx.has = (w is not None, b is not None)
        return y

    @staticmethod
    def backward(ctx, g):
        x, w, mean, rstd = ctx.saved_tensors
        dx, dw, db = K.layernorm_bwd(g if g.is_contiguous() else K.contiguous(g), x, w, mean, rstd)
        hw, hb = ctx.has
        out = [dx]
        if hw:
            out.append(dw.to(w.dtype))
        if hb:
            out.append(db.to(w.dtype if w is not None else x.dtype))
        return tuple(out)


class SwiGLUFunction(Function):
    raw = True
    amp_policy = AMPPolicy.PRESERVE

    @staticmethod
    def forward(ctx, gate, up):
        ctx.save_for_backward(gate, up)
        return K.swiglu_fwd(gate, up)

    @staticmethod
    def backward(ctx, g):
        gate, up = ctx.saved_tensors
        return K.swiglu_bwd(g if g.is_contiguous() else K.contiguous(g), gate, up)


class RoPEFunction(Function):
    """Rotate-half rotary embedding on [B, S, H, D] in one kernel (the reference composes
    ~14 launches per tensor, `models/transformers/components.py:121-179`)."""
    raw = True
    amp_policy = AMPPolicy.PRESERVE

    @staticmethod
    def forward(ctx, x, cos, sin, positions):
        ctx.save_for_backward(cos, sin, positions)
        return K.rope_fwd(x, cos, sin, positions, False)

    @staticmethod
    def backward(ctx, g):
        cos, sin, positions = ctx.saved_tensors
        return K.rope_fwd(g if g.is_contiguous() else K.contiguous(g), cos, sin, positions, True)


class FusedAttention(Function):
    """Flash attention on [B, S, H, D] tensors with native GQA (Hkv divides Hq), optional
    causal mask, any sequence length. Saves only q, k, v, o and the per-row log-sum-exp.
    Reference counterpart: `nn/attention.py:409-519` (needs Hq == Hkv, fixed S list, causal only)."""
    raw = True
    amp_policy = AMPPolicy.FP16

    @staticmethod
    def forward(ctx, q, k, v, causal, scale):
        o, lse = K.attention_fwd(q, k, v, causal, scale)
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.meta = (causal, scale)
        return o

    @staticmethod
    def backward(ctx, g):
        q, k, v, o, lse = ctx.saved_tensors
        causal, scale = ctx.meta
        return K.attention_bwd(g if g.is_contiguous() else K.contiguous(g), q, k, v, o, lse, causal, scale)


class DropoutFunction(Function):
    raw = True
    amp_policy = AMPPolicy.PRESERVE

    @staticmethod
    def forward(ctx, x, p):
        seed, off = _random.default_generator().next_philox()
        y, mask = K.dropout_mask_apply(x, p, seed, off)
        ctx.save_for_backward(mask)
        ctx.p = p
        return y

    @staticmethod
    def backward(ctx, g):
        (mask,) = ctx.saved_tensors
        return K.mul(K.mul(g, mask.to(g.dtype)), 1.0 / (1.0 - ctx.p))


# ================================ functional API ==================================
def add(a, b):
    if _is_t(a) and _is_t(b):
        return EWiseAdd.apply(a, b)
    if _is_t(a):
        return AddScalar.apply(a, b)
    return AddScalar.apply(b, a)


def sub(a, b):
    if _is_t(a) and _is_t(b):
        return EWiseSub.apply(a, b)
    if _is_t(a):
        return SubScalar.apply(a, b, False)
    return SubScalar.apply(b, a, True)


def mul(a, b):
    if _is_t(a) and _is_t(b):
        return EWiseMul.apply(a, b)
    if _is_t(a):
        return MulScalar.apply(a, b)
    return MulScalar.apply(b, a)


multiply = mul


def truediv(a, b):
    if _is_t(a) and _is_t(b):
        return EWiseDiv.apply(a, b)
    if _is_t(a):
        return DivScalar.apply(a, b, False)
    return DivScalar.apply(b, a, True)


div = divide = truediv


def floordiv(a, b):
    out = truediv(a, b)
    return Tensor._wrap(torch.floor(out._t).to(torch.int64))


def add_scalar(a, scalar):
    return AddScalar.apply(a, scalar)


def sub_scalar(a, scalar, reverse=False):
    return SubScalar.apply(a, scalar, reverse)


def mul_scalar(a, scalar):
    return MulScalar.apply(a, scalar)


def divide_scalar(a, scalar, reverse=False):
    return DivScalar.apply(a, scalar, reverse)


def pow_scalar(a, scalar, reverse=False):
    return PowScalar.apply(a, scalar, reverse)


def pow(a, b):
    if _is_t(a) and _is_t(b):
        return PowTensor.apply(a, b)
    if _is_t(a):
        return PowScalar.apply(a, b, False)
    return PowScalar.apply(b, a, True)


def _check_inplace(a):
    from .. import grad_mode
    if a.requires_grad and a.creator is None and grad_mode.is_grad_enabled():
        raise RuntimeError("a leaf Variable that requires grad is being used in an in-place operation.")


def add_inplace(a, b):
    _check_inplace(a)
    if _is_t(b):
        K.add_(a._t, b._t.to(a._t.dtype) if b._t.dtype != a._t.dtype else b._t) if b._t.shape == a._t.shape \
            else a._t.add_(b._t)
    else:
        a._t.add_(b)
    a._version += 1
    return a


def sub_inplace(a, b):
    _check_inplace(a)
    a._t.sub_(b._t if _is_t(b) else b)
    a._version += 1
    return a


def mul_inplace(a, b):
    _check_inplace(a)
    a._t.mul_(b._t if _is_t(b) else b)
    a._version += 1
    return a


def div_inplace(a, b):
    _check_inplace(a)
    a._t.div_(b._t if _is_t(b) else b)
    a._version += 1
    return a


def negate(a):
    return Negate.apply(a)


neg = negate


def sin(a):
    return Sin.apply(a)


def cos(a):
    return Cos.apply(a)


def log(a):
    return Log.apply(a)


def exp(a):
    return Exp.apply(a)


def sqrt(a):
    return Sqrt.apply(a)


def abs(a):
    return Abs.apply(a)


def sigmoid(a):
    return Sigmoid.apply(a)


def tanh(a):
    return Tanh.apply(a)


def relu(a):
    return ReLU.apply(a)


def gelu(x):
    return GELUFunction.apply(x)


def silu(x):
    return SiLUFunction.apply(x)


def swiglu(gate, up):
    return SwiGLUFunction.apply(gate, up)


def clamp(a, min_val=None, max_val=None):
    return Clamp.apply(a, min_val, max_val)


clip = clamp


def maximum(input, other):
    if not _is_t(other):
        other = Tensor._wrap(torch.full_like(input._t, other))
    return Maximum.apply(input, other)


def where(condition, x, y):
    return Where.apply(condition, x, y)


def clone(a):
    return Clone.apply(a)


def to_device(a, device):
    return ToDevice.apply(a, device)


def eq(a, b):
    return Tensor._wrap(K.compare("eq", a._t, b._t if _is_t(b) else b))


def sum(a, axis=None, keepdims=False):
    return Summation.apply(a, axis, keepdims)


summation = sum


def mean(a, axis=None, keepdims=False):
    return Mean.apply(a, axis, keepdims)


def var(a, axis=None, keepdims=False, unbiased=True):
    m = mean(a, axis, True)
    d = a - m
    sq = d * d
    if axis is None:
        n = a.numel()
    else:
        n = 1
        for ax in _axes(axis):
            n *= a.shape[ax]
    s = sum(sq, axis, keepdims)
    return s / float(_pymax(n - 1, 1) if unbiased else n)


def std(a, axis=None, keepdims=False, unbiased=True):
    return sqrt(var(a, axis, keepdims, unbiased))


def max(a, axis=None, keepdims=False):
    return Max.apply(a, axis, keepdims)


def min(a, axis=None, keepdims=False):
    return Min.apply(a, axis, keepdims)


def logsumexp(a, axis=None):
    return LogSumExp.apply(a, axis)


def argmax(a, dim=None, keepdim=False):
    return Tensor._wrap(K.argmax(a._t, dim, keepdim))


def argmin(a, dim=None, keepdim=False):
    return Tensor._wrap(K.argmax(a._t, dim, keepdim, is_min=True))


def matmul(a, b):
    return Matmul.apply(a, b)


def _shape_arg(shape):
    if len(shape) == 1 and isinstance(shape[0], (tuple, list, torch.Size)):
        return tuple(shape[0])
    return tuple(shape)


def reshape(a, *shape):
    return Reshape.apply(a, _shape_arg(shape))


def view(a, *shape):
    return Reshape.apply(a, _shape_arg(shape))


def flatten(a, start_dim=0, end_dim=None):
    return Flatten.apply(a, start_dim, -1 if end_dim is None else end_dim)


def permute(a, dims):
    return Permute.apply(a, tuple(dims))


def transpose(a, dim0=None, dim1=None, axis=None):
    if isinstance(dim0, (tuple, list)) and dim1 is None and axis is None:     # transpose(x, (d0, d1))
        axis = tuple(dim0)
    if axis is not None:
        dim0, dim1 = axis
    if dim0 is None:
        dim0, dim1 = -1, -2
    return Transpose.apply(a, dim0, dim1)


def t(a):
    return transpose(a, -1, -2) if a.ndim >= 2 else a


def contiguous(a):
    if a._t.is_contiguous():
        return a
    return Contiguous.apply(a)


def expand(a, *shape):
    return Expand.apply(a, _shape_arg(shape))


def broadcast_to(a, shape):
    return BroadcastTo.apply(a, tuple(shape))


def squeeze(tensor, dim=None):
    return Squeeze.apply(tensor, dim)


def unsqueeze(tensor, dim):
    return Unsqueeze.apply(tensor, dim)


def stack(tensors, dim=0):
    return Stack.apply(tuple(tensors), dim)


def cat(tensors, dim=0):
    return Cat.apply(tuple(tensors), dim)


def split(a, dim=0, split_size_or_sections=1):
    """Pieces of `a` along `dim`. With the default size 1 this is the reference's
    `split(a, dim)` (`nn/functional.py:2062`): one slice per index, dimension kept."""
    return Split.apply(a, split_size_or_sections, dim)


def getitem(a, index):
    return GetItem.apply(a, _raw_index(index))


def setitem(a, index, value):
    """In-place indexed assignment. If gradients are flowing, `a` is rebound to the result of an
    out-of-place SetItem node so that autograd sees the write."""
    from .. import grad_mode
    idx = _raw_index(index)
    track = grad_mode.is_grad_enabled() and (a.requires_grad or (_is_t(value) and value.requires_grad))
    if track:
        _check_inplace(a)
        out = SetItem.apply(a, value, idx) if _is_t(value) else SetItem.apply(a, value, idx)
        a._t, a.creator, a.idx, a.requires_grad = out._t, out.creator, out.idx, out.requires_grad
    else:
        K.setitem_(a._t, idx, value._t if _is_t(value) else value)
    a._version += 1
    return a


def gather(input, dim, index):
    return Gather.apply(input, dim, Tensor._wrap(_int_index(index._t)))


def scatter(input, dim, index, src):
    return Scatter.apply(input, dim, Tensor._wrap(_int_index(index._t)), src)


def scatter_add(input, dim, index, src):
    return ScatterAddFunction.apply(input, dim, Tensor._wrap(_int_index(index._t)), src)


def topk(input, k, dim=-1, largest=True, sorted=True):
    k = builtins.min(int(k), input.shape[dim]) if input.ndim else 1       # never more elements than exist
    return TopKFunction.apply(input, k, dim, largest, sorted)


def repeat_interleave(input, repeats, dim=None):
    return RepeatInterleaveFunction.apply(input, repeats, dim)


def one_hot(indices, num_classes, dtype=None):
    return Tensor._wrap(K.one_hot(indices._t, num_classes, dtype.torch_dtype if dtype is not None else torch.float32))


def embedding(weight, idx):
    cd = amp_state.dtype if (amp_state.enabled and weight._t.dtype == torch.float32) else None
    return EmbeddingFunction.apply(weight, idx, cd)


def softmax(input, dim=-1):
    return SoftmaxFunction.apply(input, dim, False)


def log_softmax(input, dim=-1):
    return SoftmaxFunction.apply(input, dim, True)


def cross_entropy(input, target, weight=None, ignore_index=-100, reduction="mean", _inplace_backward=None):
    """Softmax cross-entropy of [..., C] logits against integer class targets."""
    if reduction not in ("mean", "sum", "none"):
        raise ValueError(f"Invalid reduction mode: {reduction}")
    C = input.shape[-1]
    lead = input.shape[:-1]
    x2 = input if input.ndim == 2 else reshape(input, (-1, C))
    tgt = target._t.reshape(-1)
    if tgt.dtype not in (torch.int64, torch.int32):
        tgt = tgt.long()
    if _inplace_backward is None:
        # Safe only when the logits are an intermediate nobody else reads afterwards; callers
        # (the causal-LM heads) opt in explicitly.
        _inplace_backward = False
    out = CrossEntropyFunction.apply(x2, Tensor._wrap(tgt), weight, ignore_index, reduction, _inplace_backward)
    if reduction == "none":
        out = reshape(out, lead)
    return out


sparse_cross_entropy = cross_entropy


def rms_norm(x, weight, eps=1e-6):
    return FusedRMSNormFunction.apply(x, weight, eps)


def layer_norm(x, weight=None, bias=None, eps=1e-5):
    return FusedLayerNormFunction.apply(x, weight, bias, eps)


def rope(x, cos, sin, positions=None):
    return RoPEFunction.apply(x, cos, sin, positions)


def _fused_params(tensors, dtype):
    """Rows of several parameter matrices (or several bias vectors) stacked in one tensor of `dtype`, rebuilt only when
    one of them changed (same cache and lifetime as the per-parameter autocast copies).  Parameters whose
    low-precision copies the optimizer keeps in one stacked buffer need no kernel at all."""
    lp = stacked_shadow_of(tensors, dtype)
    if lp is not None:
        return lp
    key = ("fused", tuple(t.data_ptr() for t in tensors), tuple(t._version for t in tensors), dtype)
    hit = amp_state.cache.get(key)
    if hit is not None and all(a is b for a, b in zip(hit[0], tensors)):
        return hit[1]
    rows = builtins.sum(t.shape[0] for t in tensors)
    out = torch.empty((rows,) + tuple(tensors[0].shape[1:]), dtype=dtype, device=tensors[0].device)
    o = 0
    for t in tensors:
        K.copy_(out[o:o + t.shape[0]], t)
        o += t.shape[0]
    if amp_state.enabled:
        amp_state.cache[key] = (list(tensors), out)
    return out


def _fresh_slice(buf, start, n):
    """Rows [start, start + n) of a buffer allocated by the calling backward: a leaf may take the slice as its
    `.grad` without copying it (nothing else refers to that memory)."""
    sl = buf[start:start + n]
    sl._gb_fresh = True
    return sl


class FusedLinearFunction(Function):
    """Several linear layers that read the same input, as ONE GEMM: y = x @ cat(weights)^T + cat(biases).
    The parameters stay separate tensors (state dict and module tree are unchanged); their rows are stacked into one
    compute-dtype matrix per step, and backward runs one data-gradient GEMM and one weight-gradient GEMM whose result
    is handed back as row slices.  Replaces e.g. three projections + two gradient additions of an attention block."""
    raw = True
    amp_policy = AMPPolicy.PRESERVE

    @staticmethod
    def forward(ctx, x, weights, biases, compute_dtype):
        cd = compute_dtype if compute_dtype is not None else weights[0].dtype
        W = _fused_params(weights, cd)
        Bv = _fused_params(biases, cd) if biases else None
        if x.dtype != cd:
            x = K.to_dtype(x, cd)
        ctx.save_for_backward(x, W)
        ctx.meta = ([w.shape[0] for w in weights], weights[0].dtype, biases[0].dtype if biases else None)
        return K.linear(x, W, Bv)

    @staticmethod
    def backward(ctx, g):
        x, W = ctx.saved_tensors
        sizes, wd, bd = ctx.meta
        if g.dtype != x.dtype:
            g = K.to_dtype(g, x.dtype)
        g = g if g.is_contiguous() else K.contiguous(g)
        need = ctx.needs_input_grad
        gx = K.linear_dgrad(g, W) if need[0] else None
        stacked, accumulate = _stacked_grad_slot(ctx, 1, sizes, wd, W.shape[1])
        if stacked is not None:
            # the members' gradient slots (DDP bucket views) are adjacent in stacking order: one store into the bucket
            gW = K.linear_wgrad(g, x, out_dtype=stacked.dtype, accum=stacked if accumulate else None,
                                out=None if accumulate else stacked)
        else:
            gW = K.linear_wgrad(g, x, out_dtype=wd)
        outs, o = [gx], 0
        for n in sizes:
            outs.append(_fresh_slice(gW, o, n))
            o += n
        if bd is not None:
            gb = K.bias_grad(g, bd)
            o = 0
            for n in sizes:
                outs.append(_fresh_slice(gb, o, n))
                o += n
        return tuple(outs)


def fused_linear(x, weights, biases=None):
    """[..., sum(out_features)] = x through all of `weights` (a list of [out_i, in] parameters) at once."""
    cd = amp_state.dtype if amp_state.enabled else None
    return FusedLinearFunction.apply(x, list(weights), list(biases) if biases else [], cd)


class QKVRopeFunction(Function):
    """y [B, S, (Hq + 2 Hkv) D] from a fused q/k/v projection -> rotated q [B, S, Hq, D], rotated k and v
    [B, S, Hkv, D].  The rotary kernel reads its head slice of y in place (token-row stride = width of y); backward
    rotates the gradients back straight into their slices of one [B, S, width] buffer, so the projection's backward
    is a single pair of GEMMs with no concatenation or addition passes."""
    raw = True
    amp_policy = AMPPolicy.PRESERVE

    @staticmethod
    def forward(ctx, y, cos, sin, positions, Hq, Hkv, D):
        B, S, Nt = y.shape
        y = y if y.is_contiguous() else K.contiguous(y)
        q_in = y[..., :Hq * D].unflatten(-1, (Hq, D))
        k_in = y[..., Hq * D:(Hq + Hkv) * D].unflatten(-1, (Hkv, D))
        v_in = y[..., (Hq + Hkv) * D:].unflatten(-1, (Hkv, D))
        ctx.save_for_backward(cos, sin, positions)
        ctx.meta = (B, S, Nt, Hq, Hkv, D, y.dtype)
        fused = K.qkv_rope_split(y, cos, sin, positions, Hq, Hkv, D)      # one launch for q, k and v
        if fused is not None:
            return fused
        q = K.rope_fwd(q_in, cos, sin, positions, False)
        k = K.rope_fwd(k_in, cos, sin, positions, False)
        return q, k, K.contiguous(v_in)

    @staticmethod
    def backward(ctx, gq, gk, gv):
        cos, sin, positions = ctx.saved_tensors
        B, S, Nt, Hq, Hkv, D, dt = ctx.meta
        dev = (gq if gq is not None else gk if gk is not None else gv).device
        if all(g is not None and g.dtype == dt for g in (gq, gk, gv)):
            gs = [g if g.is_contiguous() else K.contiguous(g) for g in (gq, gk, gv)]
            dy = K.qkv_rope_merge(gs[0], gs[1], gs[2], cos, sin, positions, Hq, Hkv, D)
            if dy is not None:
                return dy
        dy = torch.empty(B, S, Nt, dtype=dt, device=dev)
        parts = ((gq, 0, Hq, True), (gk, Hq * D, Hkv, True), (gv, (Hq + Hkv) * D, Hkv, False))
        for g, off, H, rotate in parts:
            dst = dy[..., off:off + H * D].unflatten(-1, (H, D))
            if g is None:
                dst.zero_()
                continue
            g = g if g.dtype == dt else K.to_dtype(g, dt)
            if rotate:
                K.rope_fwd(g if g.is_contiguous() else K.contiguous(g), cos, sin, positions, True, out=dst)
            else:
                K.copy_(dst, g)
        return dy


class SwiGLUFusedFunction(Function):
    """silu(gate) * up where gate | up are the two column halves of one tensor (a fused gate/up projection); the
    backward writes d(gate | up) as one tensor, ready for a single pair of projection-gradient GEMMs."""
    raw = True
    amp_policy = AMPPolicy.PRESERVE

    @staticmethod
    def forward(ctx, gu):
        gu = gu if gu.is_contiguous() else K.contiguous(gu)
        ctx.save_for_backward(gu)
        return K.swiglu_fused_fwd(gu)

    @staticmethod
    def backward(ctx, g):
        (gu,) = ctx.saved_tensors
        g = g if g.dtype == gu.dtype else K.to_dtype(g, gu.dtype)
        return K.swiglu_fused_bwd(g if g.is_contiguous() else K.contiguous(g), gu)


def swiglu_fused(gate_up):
    return SwiGLUFusedFunction.apply(gate_up)


class LinearSwiGLUFunction(Function):
    """h = silu(x @ Wg^T) * (x @ Wu^T) as one node: the gate and up projections run as ONE GEMM over the stacked
    weights whose epilogue applies the activation (`K.linear_swiglu`), so the [tokens, 2 I] intermediate is written
    once (kept for backward) and never read back in the forward pass.  Backward: d(gate | up) from one SwiGLU-backward
    pass, then one data-gradient and one weight-gradient GEMM for both projections.
    Reference counterparts: `nn/modules/transformer.py` FeedFowardSwiGLU, `nn/triton_ops/silu.py:29-85`."""
    raw = True
    amp_policy = AMPPolicy.PRESERVE

    @staticmethod
    def forward(ctx, x, w_gate, w_up, compute_dtype):
        cd = compute_dtype if compute_dtype is not None else w_gate.dtype
        W = _fused_params([w_gate, w_up], cd)
        if x.dtype != cd:
            x = K.to_dtype(x, cd)
        gu, h = K.linear_swiglu(x, W)
        ctx.save_for_backward(x, W, gu)
        ctx.meta = ([w_gate.shape[0], w_up.shape[0]], w_gate.dtype)
        return h

    @staticmethod
    def backward(ctx, g):
        x, W, gu = ctx.saved_tensors
        sizes, wd = ctx.meta
        if g.dtype != gu.dtype:
            g = K.to_dtype(g, gu.dtype)
        g = g if g.is_contiguous() else K.contiguous(g)
        dgu = K.swiglu_fused_bwd(g, gu if gu.is_contiguous() else K.contiguous(gu))
        need = ctx.needs_input_grad
        gx = K.linear_dgrad(dgu, W) if need[0] else None
        stacked, accumulate = _stacked_grad_slot(ctx, 1, sizes, wd, W.shape[1])
        if stacked is not None:
            gW = K.linear_wgrad(dgu, x, out_dtype=stacked.dtype, accum=stacked if accumulate else None,
                                out=None if accumulate else stacked)
        else:
            gW = K.linear_wgrad(dgu, x, out_dtype=wd)
        return gx, _fresh_slice(gW, 0, sizes[0]), _fresh_slice(gW, sizes[0], sizes[1])


def linear_swiglu(x, w_gate, w_up):
    """silu(x @ w_gate^T) * (x @ w_up^T) for two bias-free projections of equal width."""
    cd = amp_state.dtype if amp_state.enabled else None
    return LinearSwiGLUFunction.apply(x, w_gate, w_up, cd)


class SwiGLUMLPFunction(Function):
    """The whole bias-free SwiGLU MLP, y = (silu(x Wg^T) * (x Wu^T)) Wd^T, as one node: three GEMMs forward (gate|up with
    the activation in its epilogue, down) and four backward, with no stand-alone activation pass in either direction:
    the down projection's data-gradient GEMM applies the SwiGLU backward in its epilogue (`K.dgrad_swiglu_bwd`), so
    the gradient of the hidden activation never reaches memory.
    Reference counterpart: `nn/modules/transformer.py` FeedFowardSwiGLU (three Linear modules and SiLU)."""
    raw = True
    amp_policy = AMPPolicy.PRESERVE

    @staticmethod
    def forward(ctx, x, w_gate, w_up, w_down, compute_dtype):
        cd = compute_dtype if compute_dtype is not None else w_gate.dtype
        Wgu = _fused_params([w_gate, w_up], cd)
        Wd = _cached_param_cast(w_down, cd)
        if x.dtype != cd:
            x = K.to_dtype(x, cd)
        gu, h = K.linear_swiglu(x, Wgu)
        y = K.linear(h, Wd)
        ctx.save_for_backward(x, Wgu, gu, h, Wd)
        ctx.meta = ([w_gate.shape[0], w_up.shape[0]], w_gate.dtype, w_down.dtype)
        return y

    @staticmethod
    def backward(ctx, gy):
        x, Wgu, gu, h, Wd = ctx.saved_tensors
        sizes, wd_gu, wd_d = ctx.meta
        if gy.dtype != h.dtype:
            gy = K.to_dtype(gy, h.dtype)
        gy = gy if gy.is_contiguous() else K.contiguous(gy)
        need = ctx.needs_input_grad
        # down projection: weight gradient (into its bucket slot when it has one), then data gradient + activation
        slot = _grad_slot(ctx, 3, wd_d, Wd.shape)
        if slot is None:
            gWd = K.linear_wgrad(gy, h, out_dtype=wd_d)
        else:
            buf, accumulate = slot
            gWd = K.linear_wgrad(gy, h, out_dtype=buf.dtype, accum=buf if accumulate else None,
                                 out=None if accumulate else buf)
        dgu = K.dgrad_swiglu_bwd(gy, Wd, gu if gu.is_contiguous() else K.contiguous(gu))
        gx = K.linear_dgrad(dgu, Wgu) if need[0] else None
        stacked, accumulate = _stacked_grad_slot(ctx, 1, sizes, wd_gu, Wgu.shape[1])
        if stacked is not None:
            gW = K.linear_wgrad(dgu, x, out_dtype=stacked.dtype, accum=stacked if accumulate else None,
                                out=None if accumulate else stacked)
        else:
            gW = K.linear_wgrad(dgu, x, out_dtype=wd_gu)
        return gx, _fresh_slice(gW, 0, sizes[0]), _fresh_slice(gW, sizes[0], sizes[1]), gWd


def swiglu_mlp(x, w_gate, w_up, w_down):
    """down(silu(gate(x)) * up(x)) for three bias-free projections given by their weights."""
    cd = amp_state.dtype if amp_state.enabled else None
    return SwiGLUMLPFunction.apply(x, w_gate, w_up, w_down, cd)


def qkv_rope(y, cos, sin, positions, num_heads, num_kv_heads, head_dim):
    return QKVRopeFunction.apply(y, cos, sin, positions, num_heads, num_kv_heads, head_dim)


def flash_attention(q, k, v, causal=True, scale=None):
    """q [B, S, Hq, D]; k, v [B, S, Hkv, D] -> [B, S, Hq, D]."""
    if scale is None:
        scale = 1.0 / math.sqrt(q.shape[-1])
    return FusedAttention.apply(q, k, v, causal, scale)


def scaled_dot_product_attention(q, k, v, attn_mask=None, dropout_p=0.0, is_causal=False, scale=None):
    """torch-layout SDPA: q [B, H, S, D]. Parity: reference `nn/attention.py:521-532`, but the
    causal flag is honoured and GQA needs no K/V replication."""
    if attn_mask is not None:
        s = matmul(q, transpose(k, -1, -2)) * (scale if scale is not None else 1.0 / math.sqrt(q.shape[-1]))
        s = s + attn_mask
        return matmul(softmax(s, -1), v)
    qt, kt, vt = (contiguous(transpose(x, 1, 2)) for x in (q, k, v))
    o = flash_attention(qt, kt, vt, is_causal, scale)
    return transpose(o, 1, 2)


def dropout(x, p=0.5, training=True):
    if not training or p == 0.0:
        return x
    if p >= 1.0:
        return x * 0.0
    return DropoutFunction.apply(x, p)


# ---- names the reference exports from this module, kept for drop-in imports ---------------------------------------
class Norm(Function):
    """L2 norm of all elements, sqrt(sum(a^2)).  (The reference's class of this name negates its input,
    `functional.py:2065-2080`; this is the operation the name promises.)"""
    raw = True
    amp_policy = AMPPolicy.FP32

    @staticmethod
    def forward(ctx, a):
        n = torch.sqrt(K.reduce("sum", K.mul(a, a), None, False))
        ctx.save_for_backward(a, n)
        return n

    @staticmethod
    def backward(ctx, g):
        a, n = ctx.saved_tensors
        return a * (g / torch.clamp(n, min=1e-30))


def norm(a):
    return Norm.apply(a)


View = Reshape
GetItemView = GetItem
GetItemGather = GetItem


class _FunctionalAlias:
    """`X.apply(...)` for operations that are plain functions here (no gradient flows through them)."""

    def __init__(self, fn):
        self._fn = fn

    def apply(self, *a, **k):
        return self._fn(*a, **k)


Equal = _FunctionalAlias(lambda a, b: eq(a, b))
Argmax = _FunctionalAlias(lambda a, dim=None, keepdim=False: argmax(a, dim, keepdim))
Argmin = _FunctionalAlias(lambda a, dim=None, keepdim=False: argmin(a, dim, keepdim))


def cast_fp32(x):
    """Differentiable cast to float32."""
    from ..function import cast
    return cast(x, torch.float32)


cast_to_fp32 = cast_fp32
CastFP32 = _FunctionalAlias(cast_fp32)


def cast_to_fp16(x):
    from ..function import cast
    return cast(x, torch.float16)


def sum_to_shape(data, shape):
    """Sum the broadcast dimensions of `data` so that the result has `shape` (the inverse of broadcasting)."""
    return Tensor._wrap(K.sum_to_shape(data._t if isinstance(data, Tensor) else data, tuple(shape)))


# ---- the reference's fused-op entry points (its `nn/attention.py`, `nn/layer_norm.py`, `nn/triton_ops/*`) ----------
def fused_attention(q, k, v):
    """Causal flash attention on [B, H, S, D] tensors (reference `nn/attention.py:518`); GQA needs no K/V repeat."""
    return scaled_dot_product_attention(q, k, v, is_causal=True)


def fused_layer_norm(x, weight, bias, eps=1e-6):
    """Reference `nn/layer_norm.py:212` (default eps 1e-6 there, 1e-5 in `triton_ops/layer_norm.py:232`)."""
    return FusedLayerNormFunction.apply(x, weight, bias, eps)


def fused_rmsnorm(x, weight, eps=1e-6):
    """Reference `nn/triton_ops/rmsnorm.py:242`."""
    return FusedRMSNormFunction.apply(x, weight, eps)


def safe_softmax(x, dim=-1, dtype=None):
    """Softmax that subtracts the row maximum (all softmax kernels here do); optional output dtype.
    Reference `nn/triton_ops/softmax.py:142`."""
    out = SoftmaxFunction.apply(x, dim, False)
    return out if dtype is None else out.to_dtype(dtype)


triton_softmax = safe_softmax
triton_gelu = gelu
