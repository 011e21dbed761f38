"""`Parameter` and `Module`. Parity: reference `genesis/nn/modules/module.py:15-427`.

Parameters, buffers and children are discovered by walking `__dict__` (dict / list /
tuple / Module recursion) like the reference, but every object is reported once
(the reference lists `Sequential` children twice, so optimizers step them twice).
State-dict keys follow the reference's contract: a list- or tuple-held child at
position i of attribute `attr` is keyed `attr.i.` for `ModuleList`-style containers
(`layers.0.weight`) and `i.` for `Sequential`.
"""
from collections import OrderedDict

import torch

from ...tensor import Tensor
from ...device import as_torch_device
from ...dtypes import get_dtype


class Parameter(Tensor):
    """A tensor that a Module registers as trainable. (No `__slots__`: parallel wrappers tag
    parameters with attributes such as `_no_ddp`.)"""

    def __init__(self, data, requires_grad=True):
        if isinstance(data, Tensor):
            raw = data._t
        elif isinstance(data, torch.Tensor):
            raw = data
        else:
            raw = Tensor(data, dtype=get_dtype(None))._t
        super().__init__(raw.detach() if isinstance(raw, torch.Tensor) else raw)
        self.requires_grad = requires_grad

    def __reduce__(self):
        return Tensor.__reduce__(self)


class _KeepDuplicates(set):
    """A `seen` set that never remembers: shared (tied) tensors are listed under every name."""

    def __contains__(self, item):
        return False

    def add(self, item):
        pass


def _walk(value, kind, prefix, out, seen):
    """Collect (name, object) pairs of `kind` in {'param', 'buffer', 'module'}."""
    if isinstance(value, Module):
        if kind == "module":
            if id(value) not in seen:
                seen.add(id(value))
                out.append((prefix.rstrip("."), value))
            else:
                return
        for k, v in value.__dict__.items():
            if k.startswith("_non_persistent") or k == "training":
                continue
            key = k
            if isinstance(value, ModuleContainer) and k == value._list_attr:
                # children of a container are keyed by their index alone
                _walk(v, kind, prefix, out, seen)
                continue
            if isinstance(value, ModuleContainer) and k.startswith("_alias_"):
                continue
            _walk(v, kind, f"{prefix}{key}.", out, seen)
    elif isinstance(value, Parameter):
        if kind == "param" and id(value) not in seen:
            seen.add(id(value))
            out.append((prefix.rstrip("."), value))
    elif isinstance(value, Tensor):
        if kind == "buffer" and id(value) not in seen:
            seen.add(id(value))
            out.append((prefix.rstrip("."), value))
    elif isinstance(value, dict):
        for k, v in value.items():
            _walk(v, kind, f"{prefix}{k}.", out, seen)
    elif isinstance(value, (list, tuple)):
        for i, v in enumerate(value):
            _walk(v, kind, f"{prefix}{i}.", out, seen)


class Module:
    def __init__(self):
        self.training = True

    # ---- registration -----------------------------------------------------------
    def register_buffer(self, name, buffer, persistent=True):
        object.__setattr__(self, name, buffer)
        np_set = self.__dict__.setdefault("_non_persistent_buffers", set())
        if not persistent:
            np_set.add(name)
        else:
            np_set.discard(name)

    def register_parameter(self, name, param):
        object.__setattr__(self, name, param)

    def add_module(self, name, module):
        object.__setattr__(self, name, module)

    # ---- traversal ---------------------------------------------------------------
    def named_parameters(self, prefix="", recurse=True, remove_duplicate=True):
        out = []
        if recurse:
            _walk(self, "param", prefix + "." if prefix else "", out,
                  set() if remove_duplicate else _KeepDuplicates())
        else:
            for k, v in self.__dict__.items():
                if isinstance(v, Parameter):
                    out.append(((prefix + "." if prefix else "") + k, v))
        return iter(out)

    def parameters(self):
        return [p for _, p in self.named_parameters()]

    def named_buffers(self, prefix="", recurse=True):
        out = []
        _walk(self, "buffer", prefix + "." if prefix else "", out, set())
        return iter(out)

    def buffers(self):
        return iter([b for _, b in self.named_buffers()])

    def vars(self):
        return self.parameters() + [b for _, b in self.named_buffers()]

    def named_modules(self, memo=None, prefix=""):
        out = []
        _walk(self, "module", prefix + "." if prefix else "", out, set() if memo is None else memo)
        return iter(out)

    def modules(self):
        return iter([m for _, m in self.named_modules()])

    def _children(self):
        return [m for _, m in self.named_modules() if m is not self]

    def children(self):
        out, seen = [], set()
        for v in self.__dict__.values():
            tmp = []
            if isinstance(v, Module):
                tmp = [v]
            elif isinstance(v, (list, tuple)):
                tmp = [x for x in v if isinstance(x, Module)]
            elif isinstance(v, dict):
                tmp = [x for x in v.values() if isinstance(x, Module)]
            for m in tmp:
                if id(m) not in seen:
                    seen.add(id(m))
                    out.append(m)
        return iter(out)

    def num_parameters(self):
        seen, total = set(), 0
        for p in self.parameters():
            key = (p._t.data_ptr(), p._t.numel())
            if key not in seen:
                seen.add(key)
                total += p._t.numel()
        return total

    def apply(self, fn):
        for m in list(self.modules()):
            fn(m)
        return self

    # ---- state dict ---------------------------------------------------------------
    def _non_persistent_names(self):
        names = set()
        for mname, m in self.named_modules():
            for b in m.__dict__.get("_non_persistent_buffers", ()):
                names.add(f"{mname}.{b}" if mname else b)
        return names

    def state_dict(self, destination=None, prefix="", compat=False):
        """name -> plain Tensor sharing storage. Non-persistent buffers are left out unless
        `compat=True` (the reference ignores `persistent`, `module.py:132-145`, so its strict
        loader expects e.g. the RoPE caches)."""
        sd = OrderedDict() if destination is None else destination
        skip = set() if compat else self._non_persistent_names()
        for name, p in self.named_parameters(remove_duplicate=False):
            sd[prefix + name] = Tensor._wrap(p._t)
        for name, b in self.named_buffers():
            if name not in skip:
                sd[prefix + name] = Tensor._wrap(b._t)
        for mname, m in self.named_modules():
            hook = getattr(m, "_state_dict_hook", None)
            if hook is not None:
                hook(sd, prefix + (mname + "." if mname else ""))
        return sd

    def load_state_dict(self, state_dict, strict=True):
        state_dict = dict(state_dict)
        for mname, m in self.named_modules():
            hook = getattr(m, "_load_state_dict_pre_hook", None)
            if hook is not None:
                hook(state_dict, mname + "." if mname else "")
        own_p = dict(self.named_parameters(remove_duplicate=False))
        own_b = dict(self.named_buffers())
        optional = self._non_persistent_names()
        aliases = {}
        for k in state_dict:
            # Sequential files of the reference carry both `_0.w` and `0.w` style keys.
            parts = k.split(".")
            alt = ".".join(p[1:] if (p.startswith("_") and p[1:].isdigit()) else p for p in parts)
            if alt != k:
                aliases[k] = alt
        missing = [k for k in list(own_p) + [b for b in own_b if b not in optional] if k not in state_dict]
        unexpected = [k for k in state_dict if k not in own_p and k not in own_b and aliases.get(k, k) not in own_p
                      and aliases.get(k, k) not in own_b]
        if strict and (missing or unexpected):
            raise KeyError(f"load_state_dict: missing keys {missing}, unexpected keys {unexpected}")
        for k, v in state_dict.items():
            k = k if (k in own_p or k in own_b) else aliases.get(k, k)
            tgt = own_p.get(k)
            if tgt is None:
                tgt = own_b.get(k)
            if tgt is None:
                continue
            src = v._t if isinstance(v, Tensor) else torch.as_tensor(v)
            if tuple(src.shape) != tuple(tgt._t.shape):
                if src.numel() == tgt._t.numel():
                    src = src.reshape(tgt._t.shape)
                else:
                    raise ValueError(f"size mismatch for {k}: {tuple(src.shape)} vs {tuple(tgt._t.shape)}")
            tgt._t.copy_(src.to(device=tgt._t.device, dtype=tgt._t.dtype))
            tgt._version += 1
        return missing, unexpected

    # ---- modes / movement -----------------------------------------------------------
    def train(self, mode=True):
        for m in self.modules():
            m.training = mode
        return self

    def eval(self):
        return self.train(False)

    def _apply_tensors(self, fn):
        for v in self.vars():
            new = fn(v._t)
            if new is not v._t:
                v._t = new
                v._version += 1
                if v.grad is not None:
                    v.grad._t = fn(v.grad._t)
        return self

    def to(self, *args, **kwargs):
        device = kwargs.get("device")
        dtype = kwargs.get("dtype")
        for a in args:
            if isinstance(a, str) and a.split(":")[0] not in ("cpu", "cuda"):
                dtype = a
            elif isinstance(a, (str, torch.device)) or hasattr(a, "is_cuda"):
                device = a
            else:
                dtype = a
        td = None if device is None else as_torch_device(device)
        tt = None if dtype is None else get_dtype(dtype).torch_dtype

        def conv(t):
            out = t
            if td is not None and out.device != td:
                out = out.to(td)
            if tt is not None and out.dtype.is_floating_point and out.dtype != tt:
                out = out.to(tt)
            return out
        return self._apply_tensors(conv)

    def cuda(self, device_name="cuda"):
        if isinstance(device_name, int):
            device_name = f"cuda:{device_name}"
        return self.to(device_name)

    def cpu(self):
        return self.to("cpu")

    def half(self):
        return self.to(dtype="float16")

    def bfloat16(self):
        return self.to(dtype="bfloat16")

    def float(self):
        return self.to(dtype="float32")

    def zero_grad(self):
        for p in self.parameters():
            p.grad = None

    def requires_grad_(self, flag=True):
        for p in self.parameters():
            p.requires_grad = flag
        return self

    def forward(self, *args, **kwargs):
        raise NotImplementedError

    def __call__(self, *args, **kwargs):
        return self.forward(*args, **kwargs)

    def extra_repr(self):
        return ""

    def __repr__(self):
        lines = [f"{type(self).__name__}({self.extra_repr()}"]
        for k, v in self.__dict__.items():
            if isinstance(v, Module):
                sub = repr(v).replace("\n", "\n  ")
                lines.append(f"  ({k}): {sub}")
        return lines[0] + ")" if len(lines) == 1 else "\n".join(lines) + "\n)"


class ModuleContainer(Module):
    """Base of containers whose children live in one list attribute."""
    _list_attr = "_modules_list"
