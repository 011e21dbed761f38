"""`Function` / `Context` of the dynamic autograd, with the AMP cast policy.

Parity: reference `genesis/function.py:150-283` (apply builds the graph, AMP
casting by `amp_policy`, forward runs without grad) and `:286-421` (cast
functions, cast cache for parameters).  Differences by design:

* every tensor input owns one edge slot (``None`` when it needs no gradient), so
  gradients can never be paired with the wrong input;
* built-in functions set ``raw = True`` and then receive / return plain
  ``torch.Tensor`` objects, which keeps per-op host time to a few microseconds;
  user subclasses (``raw = False``) see ``genesis_b200.Tensor`` objects as in the
  reference;
* leaf gradients run the tensor's hooks and post-accumulate hooks, which is what
  lets `DistributedDataParallel` overlap communication with backward.
"""
import os
from enum import Enum

import torch

from . import grad_mode
from .amp_state import amp_state, shadow_of


# GENESIS_NVTX=1: one NVTX range per Function forward (and "<name>.backward" per backward node), for timelines
_NVTX = os.environ.get("GENESIS_NVTX", "0") == "1" and torch.cuda.is_available()


class AMPPolicy(Enum):
    FP16 = "fp16"          # cast floating inputs to the autocast dtype
    FP32 = "fp32"          # cast floating inputs to float32
    PROMOTE = "promote"    # mixed fp32 + low precision -> fp32
    PRESERVE = "preserve"  # leave dtypes alone


_LOW = (torch.float16, torch.bfloat16)


class Context:
    __slots__ = ("saved_tensors", "needs_input_grad", "__dict__")

    def __init__(self):
        self.saved_tensors = ()
        self.needs_input_grad = ()

    def save_for_backward(self, *tensors):
        self.saved_tensors = tensors

    def release(self):
        self.saved_tensors = ()
        self.__dict__.clear()


class Edge:
    """Where one input gradient goes: a leaf tensor or (node, output index)."""
    __slots__ = ("node", "idx", "leaf")

    def __init__(self, node, idx, leaf):
        self.node = node
        self.idx = idx
        self.leaf = leaf


def _cast_raw(t, dtype):
    from .ops import dispatch as K
    return K.to_dtype(t, dtype)


class Function:
    """Base class of differentiable operations.

    Subclasses implement ``forward(ctx, *args)`` and ``backward(ctx, *grad_outputs)``.
    ``backward`` returns one gradient per *tensor* argument of ``forward`` (a single
    value or a tuple; ``None`` where no gradient exists).
    """

    amp_policy = AMPPolicy.PROMOTE
    raw = False
    keep_ctx = False   # True: the engine leaves ctx intact after backward (node may be reused)

    __slots__ = ("ctx", "edges", "n_out", "_hooks", "__weakref__")

    @staticmethod
    def forward(ctx, *args, **kwargs):
        raise NotImplementedError

    @staticmethod
    def backward(ctx, *grad_outputs):
        raise NotImplementedError

    @classmethod
    def apply(cls, *args, **kwargs):
        from .tensor import Tensor
        policy = cls.amp_policy
        st = amp_state
        # ---- AMP casting / promotion --------------------------------------------
        if st.enabled:
            if policy is AMPPolicy.FP16:
                args = _autocast_args(args, st.dtype)
            elif policy is AMPPolicy.FP32:
                args = _autocast_args(args, torch.float32)
            elif policy is AMPPolicy.PROMOTE:
                args = _promote_args(args)
        elif policy is not AMPPolicy.PRESERVE:
            args = _promote_args(args)

        # ---- collect tensor inputs ----------------------------------------------
        grad_on = grad_mode.is_grad_enabled()
        tensor_inputs = []
        for a in args:
            if isinstance(a, Tensor):
                tensor_inputs.append(a)
            elif isinstance(a, (list, tuple)) and a and isinstance(a[0], Tensor):
                tensor_inputs.extend(a)
        needs = tuple(t.requires_grad for t in tensor_inputs) if grad_on else (False,) * len(tensor_inputs)
        track = any(needs)

        node = cls.__new__(cls)
        ctx = Context()
        ctx.needs_input_grad = needs
        node.ctx = ctx

        prev = grad_on
        grad_mode._set(False)
        if _NVTX:
            torch.cuda.nvtx.range_push(cls.__name__)
        try:
            if cls.raw:
                raw_args = tuple(_unwrap(a) for a in args)
                out = cls.forward(ctx, *raw_args, **kwargs)
            else:
                out = cls.forward(ctx, *args, **kwargs)
        finally:
            grad_mode._set(prev)
            if _NVTX:
                torch.cuda.nvtx.range_pop()

        is_tuple = isinstance(out, (tuple, list))
        outs = out if is_tuple else (out,)
        results = []
        for i, o in enumerate(outs):
            if isinstance(o, torch.Tensor):
                o = Tensor._wrap(o)
            if isinstance(o, Tensor):
                if track and o._t.dtype.is_floating_point:
                    o.requires_grad = True
                    o.creator = node
                    o.idx = i
                else:
                    o.requires_grad = False
            results.append(o)

        if track:
            node.n_out = len(results)
            node.edges = tuple(
                (Edge(None, 0, t) if t.creator is None else Edge(t.creator, t.idx, None)) if need else None
                for t, need in zip(tensor_inputs, needs))
            ctx.edges = node.edges        # lets a backward see whether an input is a leaf with a gradient slot
        else:
            ctx.release()
        return tuple(results) if is_tuple else results[0]


def _unwrap(a):
    from .tensor import Tensor
    if isinstance(a, Tensor):
        return a._t
    if isinstance(a, (list, tuple)) and a and isinstance(a[0], Tensor):
        return type(a)(x._t for x in a)
    return a


def _autocast_args(args, dtype):
    from .tensor import Tensor
    out = None
    for i, a in enumerate(args):
        if isinstance(a, Tensor):
            td = a._t.dtype
            if td.is_floating_point and td != dtype and td != torch.float64:
                if out is None:
                    out = list(args)
                out[i] = cast(a, dtype)
        elif isinstance(a, (list, tuple)) and a and isinstance(a[0], Tensor):
            if any(x._t.dtype.is_floating_point and x._t.dtype != dtype for x in a):
                if out is None:
                    out = list(args)
                out[i] = type(a)(cast(x, dtype) if x._t.dtype.is_floating_point else x for x in a)
    return args if out is None else tuple(out)


def _promote_args(args):
    """Mixed float32 + float16/bfloat16 inputs are computed in float32."""
    from .tensor import Tensor
    has32 = haslow = False
    for a in args:
        if isinstance(a, Tensor):
            d = a._t.dtype
            if d == torch.float32:
                has32 = True
            elif d in _LOW:
                haslow = True
    if not (has32 and haslow):
        return args
    return tuple(cast(a, torch.float32) if isinstance(a, Tensor) and a._t.dtype in _LOW else a for a in args)


class Cast(Function):
    """dtype conversion whose backward converts the gradient back."""
    amp_policy = AMPPolicy.PRESERVE
    raw = True
    keep_ctx = True

    @staticmethod
    def forward(ctx, x, dtype, current_copy=None):
        ctx.src = x.dtype
        return current_copy if current_copy is not None else _cast_raw(x, dtype)

    @staticmethod
    def backward(ctx, g):
        return _cast_raw(g, ctx.src) if g.dtype != ctx.src else g


def cast(t, dtype):
    """Differentiable cast; parameter casts are cached for one autocast region."""
    if t._t.dtype == dtype:
        return t
    if amp_state.enabled and t.requires_grad and t.creator is None:
        key = (id(t), dtype)
        hit = amp_state.cache.get(key)
        if hit is not None and hit[0] is t and hit[2] == t._version:
            return hit[1]
        # a copy the optimizer keeps current replaces the conversion kernel
        out = Cast.apply(t, dtype, shadow_of(t._t, dtype))
        amp_state.cache[key] = (t, out, t._version)
        return out
    return Cast.apply(t, dtype)


# Names kept for API parity with the reference (`function.py:286-421`): Function subclasses with forward / backward;
# `apply` goes through `cast`, so the autocast cache and the optimizer-kept copies serve them too.
class _CastTo(Cast):
    target = None

    @staticmethod
    def forward(ctx, x, dtype=None, current_copy=None):
        raise NotImplementedError

    @classmethod
    def apply(cls, t):
        return cast(t, cls.target)


def _cast_class(name, target):
    def forward(ctx, x, dtype=None, current_copy=None):
        return Cast.forward(ctx, x, target, current_copy)
    return type(name, (_CastTo,), {"target": target, "forward": staticmethod(forward),
                                   "backward": staticmethod(Cast.backward), "__doc__": f"Differentiable cast to {target}."})


CastToFP16 = _cast_class("CastToFP16", torch.float16)
CastToBF16 = _cast_class("CastToBF16", torch.bfloat16)
CastToFP32 = _cast_class("CastToFP32", torch.float32)


def cast_to_fp16(a):
    """Differentiable cast; a tensor that already has the dtype is returned as is (keeps its creator)."""
    return cast(a, torch.float16)


def cast_to_fp32(a):
    return cast(a, torch.float32)


def cast_to_bf16(a):
    return cast(a, torch.bfloat16)


def check_dtype(value, dtype):
    """True when `value` (a tensor, or dicts / lists / tuples of them) contains a tensor of `dtype`
    (reference `function.py:130-147`)."""
    from .tensor import Tensor
    if isinstance(value, Tensor):
        return value.dtype == dtype
    if isinstance(value, dict):
        return any(check_dtype(k, dtype) or check_dtype(v, dtype) for k, v in value.items())
    if isinstance(value, (list, tuple)):
        return any(check_dtype(v, dtype) for v in value)
    return False


class AccumulateGrad:
    """Gradient sink of a leaf tensor (reference `function.py:16-60`).  The engine here keeps the leaf on the edge
    itself (`Edge.leaf`) and never builds these nodes; the class exists for code that constructs one by hand:
    `apply_grad(g)` adds `g` into `tensor.grad` and fires the tensor's hooks, like the engine does."""

    def __init__(self, tensor):
        import weakref
        self.variable = weakref.ref(tensor)
        self.next_functions = []

    def apply_grad(self, grad):
        t = self.variable()
        if t is not None:
            from .tensor import _accumulate_leaf
            _accumulate_leaf(t, grad._t if hasattr(grad, "_t") else grad, True)
