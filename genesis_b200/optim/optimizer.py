"""Optimizers. Parity: reference `genesis/optim/optimizer.py:11-150`, `optim/adamw.py:66-176`.

Every `step()` is ONE multi-tensor kernel launch over all parameters (the reference
launches once per parameter).  State is kept as `m`/`v`/`u` dicts keyed by parameter
index, the layout the reference exposes through `state_dict()`; `load_state_dict` is
real here (the reference's is a no-op, `optimizer.py:49-53`).

AMP integration: `GradScaler.step` hands `grad_scale` / `found_inf` device scalars to
the kernel, which unscales on the fly and skips the update when an overflow was
found, with no host synchronisation.
"""
import torch

from ..tensor import Tensor
from ..ops import dispatch as K


class Optimizer:
    def __init__(self, params):
        self.params = list(params)
        # set by GradScaler for one step
        self._grad_scale = None
        self._found_inf = None

    def zero_grad(self, set_to_none=True):
        for p in self.params:
            if set_to_none or p.grad is None:
                p.grad = None
            else:
                K.fill_(p.grad._t, 0)

    reset_grad = zero_grad

    def step(self):
        raise NotImplementedError

    _STATE_TENSORS = ("m", "v", "u")

    def state_dict(self):
        out = {}
        for k, v in self.__dict__.items():
            if k == "params" or k.startswith("_"):
                continue
            if k in self._STATE_TENSORS:
                out[k] = {i: Tensor._wrap(t) for i, t in v.items()}
            else:
                out[k] = v
        return out

    def load_state_dict(self, state_dict):
        state = state_dict
        for k, v in state.items():
            if k in self._STATE_TENSORS:
                cur = {}
                for i, t in v.items():
                    raw = t._t if isinstance(t, Tensor) else torch.as_tensor(t)
                    p = self.params[int(i)]._t
                    cur[int(i)] = raw.to(device=p.device, dtype=torch.float32).clone()
                setattr(self, k, cur)
            elif k != "params":
                setattr(self, k, v)

    def _touched(self, idx):
        """Book-keeping after an in-place update of parameters `idx` by a kernel: version counters (the framework's
        and torch's, which key the autocast caches) and the validity stamp of low-precision copies."""
        ps = []
        for i in idx:
            p = self.params[i]
            p._version += 1
            ps.append(p._t)
        try:
            torch.autograd.graph.increment_version(ps)
        except (AttributeError, TypeError):               # older torch: one tensor per call, or absent
            for t in ps:
                try:
                    torch.autograd.graph.increment_version(t)
                except AttributeError:
                    break
        ents = getattr(self, "_shadow_entries", None)
        if ents:
            for i in idx:
                e = ents.get(i)
                if e is not None:
                    e.version = self.params[i]._version

    def _active(self):
        idx = [i for i, p in enumerate(self.params) if p.grad is not None]
        return idx

    def _state(self, store, i):
        t = store.get(i)
        if t is None:
            p = self.params[i]._t
            t = torch.zeros(p.shape, dtype=torch.float32 if p.dtype.is_floating_point else p.dtype,
                            device=p.device)
            store[i] = t
        return t


class SGD(Optimizer):
    """u = momentum*u + (1-momentum)*(g + wd*p); p -= lr*u."""

    def __init__(self, params, lr=0.01, momentum=0.0, weight_decay=0.0):
        super().__init__(params)
        self.lr, self.momentum, self.weight_decay = lr, momentum, weight_decay
        self.u = {}

    def step(self):
        idx = self._active()
        if not idx:
            return
        ps = [self.params[i]._t for i in idx]
        gs = [self.params[i].grad._t for i in idx]
        us = [self._state(self.u, i) for i in idx]
        K.sgd_step(ps, gs, us, self.lr, self.momentum, self.weight_decay)
        self._touched(idx)


class _AdamBase(Optimizer):
    decoupled = True
    _fused_amp = True   # the kernel takes grad_scale / found_inf device scalars (see GradScaler.step)

    def __init__(self, params, lr, beta1, beta2, eps, weight_decay):
        super().__init__(params)
        self.lr, self.beta1, self.beta2, self.eps, self.weight_decay = lr, beta1, beta2, eps, weight_decay
        self.t = 0
        self.m, self.v = {}, {}
        self._shadows = None
        # capturable mode: learning rate, bias corrections and step count live in a device vector that the kernel
        # advances, so a CUDA graph of the step can be replayed (see `genesis_b200.cuda.graphs.GraphedTrainStep`)
        self._dyn = None
        self._dyn_lr = None

    def enable_shadows(self, dtype, groups=None, transposed="auto"):
        """Keep a `dtype` (bf16 / fp16) copy of every floating-point parameter current from inside the optimizer
        kernel, so that `autocast` finds the low-precision weights ready instead of converting all of them every
        step.  `groups`: lists of parameters that some layer multiplies as one stacked matrix (q/k/v, gate/up); their
        copies are row slices of one buffer, which the fused projection then uses as is.  Costs 2 bytes per
        parameter.  A parameter changed by anything but this optimizer falls back to the conversion until the next
        step refreshes its copy.  `transposed`: also keep a [in, out] twin of 2-D weight copies (refreshed by a tiled
        transpose after each step), which the data-gradient GEMMs read instead of the [out, in] copy, so that both
        operands are contiguous along the contraction: "auto" for the weights whose layer asks for one
        (`Parameter.wants_transposed_copy`, set by the SwiGLU MLP for its down projection, whose fused backward needs
        it), True for every 2-D weight, False for none.  Costs 2 more bytes per twinned weight element.  Measured on
        Qwen2.5-0.5B (8 x 2048, one B200): 77.0 ms per step with "auto", 79.0 with True (the plain data-gradient GEMMs
        run as fast on the [out, in] copy, so the 73 extra transposes per step only cost), 78.5 with False."""
        from ..amp_state import ShadowEntry, shadows
        from ..dtypes import get_dtype
        td = get_dtype(dtype).torch_dtype
        index = {id(p): i for i, p in enumerate(self.params)}
        self._shadows, self._shadow_entries = {}, {}
        self._transposed = []                       # (copy [N, K], twin [K, N]) pairs refreshed after every step
        grouped = set()
        for members in (groups or []):
            ps = [p for p in members if id(p) in index]
            if len(ps) != len(members) or any(p._t.dtype != torch.float32 or not p._t.is_contiguous() for p in ps) \
                    or any(p._t.shape[1:] != ps[0]._t.shape[1:] for p in ps) or any(id(p) in grouped for p in ps):
                continue
            rows = sum(p._t.shape[0] for p in ps)
            buf = torch.empty((rows,) + tuple(ps[0]._t.shape[1:]), dtype=td, device=ps[0]._t.device)
            ents, o = [], 0
            group = (ents, buf)
            for p in ps:
                lp = buf[o:o + p._t.shape[0]]
                o += p._t.shape[0]
                lp.copy_(p._t)
                e = ShadowEntry(p, lp, group)
                ents.append(e)
                grouped.add(id(p))
                self._register_shadow(index[id(p)], e, shadows)
            if transposed is True and buf.dim() == 2:
                self._add_transposed(buf)
        for i, p in enumerate(self.params):
            if id(p) in grouped or p._t.dtype != torch.float32 or not p._t.is_contiguous() or p._t.numel() == 0:
                continue
            e = ShadowEntry(p, p._t.to(td), None)
            self._register_shadow(i, e, shadows)
            want = transposed is True or (transposed == "auto" and getattr(p, "wants_transposed_copy", False))
            if want and e.lp.dim() == 2 and min(e.lp.shape) >= 64:
                self._add_transposed(e.lp)
        return self

    def _add_transposed(self, lp):
        from ..amp_state import transposed as registry
        twin = torch.empty(lp.shape[1], lp.shape[0], dtype=lp.dtype, device=lp.device)
        if lp.is_cuda:
            if K.transpose_into(twin, lp) is NotImplemented:
                return
        else:
            twin.copy_(lp.t())
        self._transposed.append((lp, twin))
        registry[lp.data_ptr()] = twin

    def _refresh_transposed(self):
        for lp, twin in getattr(self, "_transposed", ()):
            if lp.is_cuda:
                K.transpose_into(twin, lp)
            else:
                twin.copy_(lp.t())

    def _register_shadow(self, i, entry, registry):
        self._shadows[i] = entry.lp
        self._shadow_entries[i] = entry
        registry[entry.param._t.data_ptr()] = entry

    def disable_shadows(self):
        from ..amp_state import shadows
        from ..amp_state import transposed as registry
        for e in (getattr(self, "_shadow_entries", None) or {}).values():
            if shadows.get(e.param._t.data_ptr()) is e:
                del shadows[e.param._t.data_ptr()]
        for lp, _ in getattr(self, "_transposed", ()):
            registry.pop(lp.data_ptr(), None)
        self._shadows, self._shadow_entries, self._transposed = None, {}, []

    def make_capturable(self):
        """Move the step-dependent scalars to the device. Idempotent; needs CUDA parameters."""
        if self._dyn is None:
            dev = self.params[0]._t.device
            if dev.type != "cuda":
                raise RuntimeError("capturable optimizer state needs CUDA parameters")
            self._dyn = torch.tensor([self.lr, 1.0 - self.beta1 ** max(self.t, 1), 1.0 - self.beta2 ** max(self.t, 1),
                                      float(self.t)], dtype=torch.float32, device=dev)
            self._dyn_lr = self.lr
        return self

    def load_state_dict(self, state_dict):
        state = state_dict
        super().load_state_dict(state)
        if self._dyn is not None:                 # device copy of the step count and learning rate follows the host
            self._dyn[3:4].fill_(float(self.t))
            self._dyn[0:1].fill_(float(self.lr))
            self._dyn_lr = self.lr

    def _sync_lr(self):
        """Write a changed host learning rate into the device vector (outside a capture)."""
        if self._dyn is not None and self._dyn_lr != self.lr:
            self._dyn[0:1].fill_(float(self.lr))
            self._dyn_lr = self.lr

    def steps_applied(self):
        """Number of updates actually applied.  With a GradScaler the steps an overflow cancelled do not count; the
        exact figure then lives on the device (this reads it back and brings the host's `t` in line)."""
        if self._dyn is not None:
            self.t = int(round(float(self._dyn[3].item())))
        return self.t

    def state_dict(self):
        if self._dyn is not None and not torch.cuda.is_current_stream_capturing():
            self.steps_applied()
        return super().state_dict()

    def step(self):
        idx = self._active()
        if not idx:
            return
        if self._found_inf is not None and self._dyn is None and self.params[idx[0]]._t.is_cuda:
            # a step the overflow flag may cancel on the device: count steps there too, so that a cancelled step
            # does not advance the bias corrections (the host cannot know without reading the flag back)
            self.make_capturable()
        elif self._found_inf is not None and not self.params[idx[0]]._t.is_cuda \
                and float(self._found_inf.item()) != 0.0:
            return                                # cancelled step (host tensors: the flag is read here)
        self.t += 1
        if self._dyn is not None and not torch.cuda.is_current_stream_capturing():
            self._sync_lr()
        # parameters whose gradient all-reduce a data-parallel wrapper left in flight (`_late_join`) are updated in a
        # second launch, after the join: the first launch runs under the tail of the communication
        late = [i for i in idx if getattr(self.params[i], "_late_join", None) is not None]
        late_set = set(late)
        parts = [idx] if not late or len(late) == len(idx) else [[i for i in idx if i not in late_set], late]
        for n, part in enumerate(parts):
            if late and (n == len(parts) - 1):
                for j in {id(f): f for f in (self.params[i]._late_join for i in late)}.values():
                    if j is not None:
                        j()
            ps = [self.params[i]._t for i in part]
            gs = [self.params[i].grad._t for i in part]
            ms = [self._state(self.m, i) for i in part]
            vs = [self._state(self.v, i) for i in part]
            sh = None if self._shadows is None else [self._shadows.get(i) for i in part]
            K.adamw_step(ps, gs, ms, vs, self.lr, self.beta1, self.beta2, self.eps, self.weight_decay, self.t,
                         self.decoupled, self._grad_scale, self._found_inf, sh, self._dyn, advance=(n == 0))
        if self._shadows is not None:
            self._refresh_transposed()
        self._touched(idx)


class Adam(_AdamBase):
    """Adam with L2 weight decay folded into the gradient."""
    decoupled = False

    def __init__(self, params, lr=0.01, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.0):
        super().__init__(params, lr, beta1, beta2, eps, weight_decay)


class AdamW(_AdamBase):
    """AdamW with decoupled weight decay. `fused` is accepted for API parity: the CUDA path is
    always the fused multi-tensor kernel, the CPU path always plain math."""
    decoupled = True

    def __init__(self, params, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01, fused=True,
                 betas=None):
        if betas is not None:
            beta1, beta2 = betas
        super().__init__(params, lr, beta1, beta2, eps, weight_decay)
        self.fused = fused
