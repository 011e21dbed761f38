"""`Tensor`: an autograd-carrying handle over a `torch.Tensor`, and the backward engine.

Parity: reference `genesis/tensor.py:23-129` (attributes), `:189-377` (backward:
topological order over the creator graph, gradients summed per output, saved
tensors freed as soon as a node has run), `:379-486` (`to/cpu/cuda/numpy`),
`:778-828` (pickle through `_rebuild_tensor(numpy, dtype_name, requires_grad)`),
`:831-880` (`genesis.tensor`).  Storage, strides, views and host transfer are
torch's; autograd is this module's own (torch.autograd is never used).
"""
import numpy as np
import torch

from . import grad_mode
from .device import Device, as_torch_device
from .dtypes import DType, get_dtype, bfloat16 as _bf16


def _to_torch(data, dtype, device):
    """Python / numpy / torch payload -> torch.Tensor of `dtype` on `device`."""
    td = dtype.torch_dtype
    if isinstance(data, Tensor):
        data = data._t
    if isinstance(data, torch.Tensor):
        return data.to(device=device, dtype=td)
    if isinstance(data, np.ndarray):
        if data.dtype == np.float64 and td != torch.float64:
            data = data.astype(np.float32)
        t = torch.from_numpy(np.ascontiguousarray(data).reshape(data.shape))
        return t.to(device=device, dtype=td)
    return torch.tensor(data, dtype=td, device=device)


class Tensor:
    __slots__ = ("_t", "requires_grad", "grad", "creator", "idx", "_hooks", "_post_hooks",
                 "_version", "_grad_buf", "__weakref__")

    def __init__(self, data, dtype=None, device=None, requires_grad=False):
        if isinstance(data, torch.Tensor) and dtype is None and device is None:
            self._t = data
        else:
            self._t = _to_torch(data, get_dtype(dtype), as_torch_device(device))
        self.requires_grad = requires_grad
        self.grad = None
        self.creator = None
        self.idx = 0
        self._hooks = None
        self._post_hooks = None
        self._version = 0
        self._grad_buf = None

    @classmethod
    def _wrap(cls, t, requires_grad=False):
        obj = Tensor.__new__(Tensor)
        obj._t = t
        obj.requires_grad = requires_grad
        obj.grad = None
        obj.creator = None
        obj.idx = 0
        obj._hooks = None
        obj._post_hooks = None
        obj._version = 0
        obj._grad_buf = None
        return obj

    # ---- metadata ---------------------------------------------------------------
    @property
    def shape(self):
        return tuple(self._t.shape)

    @property
    def dtype(self):
        return get_dtype(self._t.dtype)

    @property
    def device(self):
        return Device(self._t.device)

    @property
    def ndim(self):
        return self._t.dim()

    @property
    def is_leaf(self):
        return self.creator is None

    @property
    def grad_fn(self):
        return self.creator

    @property
    def is_view(self):
        return self._t._base is not None

    @property
    def base(self):
        b = self._t._base
        return None if b is None else Tensor._wrap(b)

    @property
    def offset(self):
        return self._t.storage_offset()

    def storage_offset(self):
        return self._t.storage_offset()

    @property
    def strides(self):
        return tuple(self._t.stride())

    def stride(self, dim=None):
        return tuple(self._t.stride()) if dim is None else self._t.stride(dim)

    def size(self, dim=None):
        return tuple(self._t.shape) if dim is None else self._t.shape[dim]

    def dim(self):
        return self._t.dim()

    def numel(self):
        return self._t.numel()

    def element_size(self):
        return self._t.element_size()

    def is_floating_point(self):
        return self._t.dtype.is_floating_point

    def is_contiguous(self):
        return self._t.is_contiguous()

    def data_ptr(self):
        return self._t.data_ptr()

    @property
    def is_cuda(self):
        return self._t.is_cuda

    @property
    def __cuda_array_interface__(self):
        return self._t.__cuda_array_interface__

    # ---- data aliasing ----------------------------------------------------------
    @property
    def data(self):
        """Detached alias sharing storage (no graph, no grad)."""
        return Tensor._wrap(self._t)

    @data.setter
    def data(self, value):
        self._t = value._t if isinstance(value, Tensor) else value
        self._version += 1

    def detach(self):
        return Tensor._wrap(self._t)

    def requires_grad_(self, flag=True):
        self.requires_grad = flag
        return self

    def clone(self):
        from .nn import functional as F
        return F.clone(self)

    def copy_(self, other):
        src = other._t if isinstance(other, Tensor) else _to_torch(other, self.dtype, self._t.device)
        from .ops import dispatch as K
        K.copy_(self._t, src)
        self._version += 1
        return self

    def fill_(self, value):
        from .ops import dispatch as K
        K.fill_(self._t, value)
        self._version += 1
        return self

    def zero_(self):
        return self.fill_(0)

    # ---- device / dtype movement ------------------------------------------------
    def to(self, *args, **kwargs):
        device = kwargs.get("device")
        dtype = kwargs.get("dtype")
        for a in args:
            if isinstance(a, (Device, torch.device)):
                device = a
            elif isinstance(a, (DType, torch.dtype)):
                dtype = a
            elif isinstance(a, str):
                if a.split(":")[0] in ("cpu", "cuda"):
                    device = a
                else:
                    dtype = a
            elif isinstance(a, Tensor):
                device, dtype = a._t.device, a._t.dtype
        out = self
        if dtype is not None and get_dtype(dtype).torch_dtype != self._t.dtype:
            out = out.to_dtype(dtype)
        if device is not None:
            td = as_torch_device(device)
            if td != out._t.device:
                from .nn import functional as F
                out = F.to_device(out, td)
        return out

    def to_dtype(self, dtype):
        from .function import cast
        return cast(self, get_dtype(dtype).torch_dtype)

    def cpu(self):
        return self.to("cpu")

    def cuda(self, index=None):
        return self.to(f"cuda:{index}" if index is not None else "cuda")

    def numpy(self):
        if self.requires_grad:
            raise RuntimeError("Can't call numpy() on Tensor that requires grad. Use tensor.detach().numpy() instead.")
        return self._numpy()

    def _numpy(self):
        t = self._t.detach()
        if t.dtype == torch.bfloat16:
            t = t.float()
        return t.cpu().numpy()

    def tolist(self):
        return self._numpy().tolist()

    def item(self):
        v = self._t.item()
        if self._t.is_cuda:
            # the host is synchronised here anyway: surface what the native kernels recorded (an expired
            # bounded wait, an index that was out of range and skipped) at the point the user reads a result
            from .ops import native
            if native._status:
                native.check_status(self._t.device)
        return v

    def __float__(self):
        return float(self._t.item())

    def __int__(self):
        return int(self._t.item())

    def __bool__(self):
        if self._t.numel() != 1:
            raise RuntimeError("Boolean value of Tensor with more than one value is ambiguous")
        return bool(self._t.item())

    def __index__(self):
        return int(self._t.item())

    def all(self, dim=None, keepdim=False):
        """Whether all elements are non-zero: a bool tensor (0-d without `dim`; `bool(x.all())` works).
        Parity: reference `genesis/tensor.py:565-600`."""
        t = self._t if self._t.dtype == torch.bool else (self._t != 0)
        if dim is None:
            return Tensor._wrap(t.all())
        dims = (dim,) if isinstance(dim, int) else tuple(dim)
        for d in sorted((x % t.dim() for x in dims), reverse=True):
            t = t.all(dim=d, keepdim=keepdim)
        return Tensor._wrap(t)

    def any(self, dim=None, keepdim=False):
        """Whether any element is non-zero (see `all`).  Parity: reference `genesis/tensor.py:611-635`."""
        t = self._t if self._t.dtype == torch.bool else (self._t != 0)
        if dim is None:
            return Tensor._wrap(t.any())
        dims = (dim,) if isinstance(dim, int) else tuple(dim)
        for d in sorted((x % t.dim() for x in dims), reverse=True):
            t = t.any(dim=d, keepdim=keepdim)
        return Tensor._wrap(t)

    def __hash__(self):
        return id(self)

    def __iter__(self):
        for i in range(len(self)):
            yield self[i]

    def __repr__(self):
        extra = ", requires_grad=True" if self.requires_grad else ""
        body = repr(self._t.detach().cpu()).replace("tensor(", "Tensor(", 1)
        if body.endswith(")"):
            body = body[:-1] + f", device='{self.device}'{extra})"
        return body

    # ---- pickling: the on-disk checkpoint format --------------------------------
    def __reduce__(self):
        t = self._t.detach()
        name = get_dtype(t.dtype).name
        arr = (t.float() if t.dtype == torch.bfloat16 else t).cpu().numpy()
        return (_rebuild_tensor, (arr, name, bool(self.requires_grad)))

    # ---- hooks ------------------------------------------------------------------
    def register_hook(self, fn):
        """`fn(grad) -> grad | None`, called when this tensor's gradient is ready."""
        if self._hooks is None:
            self._hooks = []
            if self.creator is not None:
                # non-leaf: the engine looks hooks up on the producing node, per output index
                table = getattr(self.creator, "_hooks", None)
                if table is None:
                    table = self.creator._hooks = {}
                table[self.idx] = self._hooks
        self._hooks.append(fn)
        return _HookHandle(self._hooks, fn)

    def register_post_accumulate_grad_hook(self, fn):
        """`fn(tensor)`, called after a leaf's `.grad` has been updated."""
        if self._post_hooks is None:
            self._post_hooks = []
        self._post_hooks.append(fn)
        return _HookHandle(self._post_hooks, fn)

    def apply_hooks(self, grad):
        if self._hooks:
            for h in self._hooks:
                r = h(grad)
                if r is not None:
                    grad = r
        return grad

    def set_creator(self, creator, idx=0):
        self.creator = creator
        self.idx = idx

    # ---- autograd ---------------------------------------------------------------
    def backward(self, out_grad=None, retain_graph=False):
        if not self.requires_grad:
            raise RuntimeError("element 0 of tensors does not require grad and does not have a grad_fn")
        if out_grad is None:
            if self._t.numel() != 1:
                raise RuntimeError("grad can be implicitly created only for scalar outputs")
            g = torch.ones_like(self._t)
        else:
            g = out_grad._t if isinstance(out_grad, Tensor) else _to_torch(out_grad, self.dtype, self._t.device)
        from .amp_state import amp_state
        saved_amp = amp_state.enabled
        amp_state.enabled = False
        prev = grad_mode.is_grad_enabled()
        grad_mode._set(False)
        _adopted.clear()
        try:
            if self.creator is None:
                _accumulate_leaf(self, g)
            else:
                _run_backward(self, g, retain_graph)
        finally:
            grad_mode._set(prev)
            amp_state.enabled = saved_amp
        for cb in list(_backward_end_callbacks):
            cb()


# Callables run after every `Tensor.backward` (DistributedDataParallel joins its
# communication stream here).
_backward_end_callbacks = []


class _HookHandle:
    def __init__(self, lst, fn):
        self._lst, self._fn = lst, fn

    def remove(self):
        try:
            self._lst.remove(self._fn)
        except ValueError:
            pass


_adopted = set()   # data pointers adopted as leaf gradients during the current backward pass


class RowScatterGrad:
    """Gradient of a row lookup (embedding) kept as (row indices, row gradients) until it reaches its leaf: added to
    a gradient that already exists (a tied output projection contributed first, or gradient accumulation) by one
    scatter-add in place, instead of materialising a zero-filled [num_rows, D] tensor and adding two dense tensors.
    Anything that needs a dense tensor calls `dense()`."""
    __slots__ = ("rows", "idx", "num_rows", "dtype")

    def __init__(self, rows, idx, num_rows, dtype):
        self.rows, self.idx, self.num_rows, self.dtype = rows, idx, num_rows, dtype

    def dense(self):
        from .ops import dispatch as K
        return K.embedding_bwd(self.rows, self.idx, self.num_rows, self.dtype)

    def add_into(self, acc):
        from .ops import dispatch as K
        if acc.dtype == torch.float32 and acc.is_contiguous() and acc.dim() == 2:
            K.embedding_bwd_into(acc, self.rows, self.idx)
        elif acc.is_cuda and acc.is_contiguous() and acc.dim() == 2 and K.index_add_rows_(acc, self.rows, self.idx):
            pass                                   # 16-bit accumulator (a 16-bit gradient slot): atomic adds in place
        else:
            K.add_(acc, self.dense().to(acc.dtype).reshape(acc.shape))


def _accumulate_leaf(t, g, fire_post_hooks=True):
    """Leaf gradient: tensor hooks, accumulation into `.grad`, post-accumulate hooks (`fire_post_hooks=False`
    while further contributions to the same leaf are still to come in this backward pass)."""
    if isinstance(g, RowScatterGrad):
        target = None
        if not t._hooks and g.num_rows == t._t.shape[0]:
            if t.grad is not None:
                target = t.grad._t
            elif t._grad_buf is not None:                  # preallocated slot (DDP bucket view)
                target = t._grad_buf
                target.zero_()
                t.grad = Tensor._wrap(target)
        if target is None:
            g = g.dense()
        else:
            g.add_into(target)
            if fire_post_hooks and t._post_hooks:
                for h in t._post_hooks:
                    h(t)
            return
    if t._hooks:
        gw = t.apply_hooks(Tensor._wrap(g))
        g = gw._t
    from .ops import dispatch as K
    buf = t._grad_buf
    in_slot = buf is not None and g.data_ptr() == buf.data_ptr() and g.dtype == buf.dtype \
        and g.numel() == buf.numel()
    # a preallocated slot may be narrower than the parameter (DDP's 16-bit wire format): gradients are brought to
    # the slot's dtype, not the parameter's
    want = buf.dtype if buf is not None and (t.grad is None or t.grad._t.data_ptr() == buf.data_ptr()) else t._t.dtype
    if not in_slot and g.dtype != want:
        g = K.to_dtype(g, want)
    if g.shape != t._t.shape:
        g = g.reshape(t._t.shape) if g.numel() == t._t.numel() else g.sum_to_size(t._t.shape)
    if in_slot:
        # the producing kernel already wrote (or accumulated) into the preallocated slot
        if t.grad is None:
            t.grad = Tensor._wrap(buf)
        elif t.grad._t.data_ptr() != buf.data_ptr():
            K.add_(t.grad._t, g)
    elif t.grad is None:
        if buf is not None:          # preallocated slot (DDP bucket view): write in place
            K.copy_(buf, g)
            t.grad = Tensor._wrap(buf)
        else:
            # `.grad` must own its memory: views / broadcast (stride-0) gradients and a tensor that
            # another leaf already took in this pass are copied, everything else is adopted as is.
            # (a Function may mark contiguous slices of a buffer it has just allocated as `_gb_fresh`: the row
            # slices of a fused weight gradient are owned by nobody else and need no copy)
            key = g.data_ptr()
            if (g._base is not None and not getattr(g, "_gb_fresh", False)) or not g.is_contiguous() \
                    or key in _adopted:
                g = K.clone(g)
            else:
                _adopted.add(key)
            t.grad = Tensor._wrap(g)
    else:
        K.add_(t.grad._t, g)
    if fire_post_hooks and t._post_hooks:
        for h in t._post_hooks:
            h(t)


def _topo(root_node):
    """Reverse-topological order (root first) by iterative DFS over creator edges."""
    order, seen = [], set()
    stack = [(root_node, 0)]
    while stack:
        node, i = stack.pop()
        if i == 0:
            if id(node) in seen:
                continue
            seen.add(id(node))
        edges = node.edges
        n = len(edges)
        while i < n:
            e = edges[i]
            i += 1
            if e is not None and e.node is not None and id(e.node) not in seen:
                stack.append((node, i))
                stack.append((e.node, 0))
                break
        else:
            order.append(node)
    order.reverse()
    return order


def _run_backward(root, g, retain_graph):
    from .ops import dispatch as K
    from . import function as _fn
    order = _topo(root.creator)
    pending = {id(root.creator): {root.idx: g}}
    # A leaf used several times in the graph (tied weights) is accumulated several times; its post-accumulate
    # hooks (DDP's "gradient is final" signal) must fire once, after the last contribution.
    uses = {}
    for node in order:
        for e in node.edges:
            if e is not None and e.leaf is not None and e.leaf._post_hooks:
                uses[id(e.leaf)] = uses.get(id(e.leaf), 0) + 1
    for node in order:
        slot = pending.pop(id(node), None)
        if slot is None:
            continue
        n_out = node.n_out
        ctx = node.ctx
        cls = type(node)
        if n_out == 1:
            gouts = (slot.get(0),)
        else:
            gouts = tuple(slot.get(i) for i in range(n_out))
        hooks = getattr(node, "_hooks", None)
        if hooks:
            gl = list(gouts)
            for i, fns in hooks.items():
                if gl[i] is not None:
                    gw = Tensor._wrap(gl[i])
                    for fn in fns:
                        r = fn(gw)
                        if r is not None:
                            gw = r
                    gl[i] = gw._t
            gouts = tuple(gl)
        if _fn._NVTX:
            torch.cuda.nvtx.range_push(cls.__name__ + ".backward")
        if cls.raw:
            res = cls.backward(ctx, *gouts)
        else:
            res = cls.backward(ctx, *[None if x is None else Tensor._wrap(x) for x in gouts])
        if _fn._NVTX:
            torch.cuda.nvtx.range_pop()
        if not retain_graph and not cls.keep_ctx:
            ctx.release()
        if not isinstance(res, (tuple, list)):
            res = (res,)
        edges = node.edges
        for e, gi in zip(edges, res):
            if e is None or gi is None:
                continue
            if isinstance(gi, Tensor):
                gi = gi._t
            if e.leaf is not None:
                left = uses.get(id(e.leaf), 1) - 1
                uses[id(e.leaf)] = left
                _accumulate_leaf(e.leaf, gi, left <= 0)
            else:
                if isinstance(gi, RowScatterGrad):
                    gi = gi.dense()
                d = pending.get(id(e.node))
                if d is None:
                    pending[id(e.node)] = {e.idx: gi}
                else:
                    cur = d.get(e.idx)
                    if cur is None:
                        d[e.idx] = gi
                    else:
                        if cur.dtype != gi.dtype:
                            gi = gi.to(cur.dtype)
                        d[e.idx] = K.add(cur, gi)
        del slot, gouts, res


def _rebuild_tensor(numpy_data, dtype_name, requires_grad):
    """Unpickle hook of the checkpoint format: always produces a CPU tensor."""
    dt = get_dtype(dtype_name)
    t = torch.from_numpy(np.ascontiguousarray(numpy_data)).to(dt.torch_dtype)
    return Tensor._wrap(t, requires_grad=bool(requires_grad))


def tensor(data, dtype=None, device=None, requires_grad=False):
    """Create a tensor from data; `dtype=None` means float32 whatever the payload
    (reference `tensor.py:845-848`)."""
    if isinstance(data, Tensor):
        data = data._t
    return Tensor(data, dtype=get_dtype(dtype), device=device if device is not None else "cpu",
                  requires_grad=requires_grad)


def make_tensor(data, dtype=None, device=None, shape=None):
    t = tensor(data, dtype, device)
    if shape is not None:
        t._t = t._t.reshape(shape)
    return t


def ones_like(tensor):
    """Tensor of ones with the shape, dtype and device of `tensor` (module-level helper of the reference's tensor.py)."""
    from . import init
    return init.ones_like(tensor)
