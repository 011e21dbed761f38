"""`DistributedDataParallel` with bucketed, overlapped, fused gradient all-reduce.

API parity: reference `genesis/nn/parallel.py:19-209` (constructor arguments, `.module` /
`.model`, delegation of `state_dict` & co., `__getattr__` fall-through, initial broadcast
from rank 0, the `DDP: Initialized model on rank r/w` line).  The reference registers one
blocking NCCL all-reduce per parameter in a tensor hook that its backward engine never
fires (`genesis/function.py:33-44`); here:

* parameters are grouped into buckets (default 25 MB, reverse registration order, so the
  first bucket to complete holds the last layers' gradients);
* every gradient is written straight into its slot of the bucket's flat buffer
  (`Tensor._grad_buf`), which on CUDA lives in the symmetric heap;
* when the last gradient of bucket i has been accumulated (post-accumulate hook) and
  buckets 0..i-1 are launched, the bucket's all-reduce is enqueued on a communication
  stream, overlapping the rest of backward;
* on CUDA the all-reduce is one kernel that pulls the rank's slice from all peers over
  NVLink, accumulates in float32, multiplies by inv_scale/world (AMP unscale), raises the
  overflow flag on Inf/NaN, and pushes the result into every peer's buffer — no NCCL call;
  on CPU ranks (gloo) the same bucket logic runs over `torch.distributed.all_reduce`;
* `no_sync()` accumulates locally for gradient accumulation.
"""
import contextlib
import os

import torch
import torch.distributed as tdist

from ..tensor import Tensor, _backward_end_callbacks
from ..distributed import process_group as pg
from ..distributed import symm
from ..distributed.collectives import comm_mode
from .modules.module import Module


class _Bucket:
    __slots__ = ("index", "params", "offsets", "numel", "dtype", "flat", "symm_buf", "pending", "launched",
                 "ready_event", "wire", "wire_dtype")

    def __init__(self, index, dtype):
        self.index, self.dtype = index, dtype
        self.params, self.offsets = [], []
        self.numel = 0
        self.flat = None
        self.symm_buf = None
        self.wire = None            # 16-bit view of the symmetric buffer when gradients cross NVLink in 16 bits
        self.wire_dtype = None
        self.pending = 0
        self.launched = False
        self.ready_event = None


class DistributedDataParallel(Module):
    def __init__(self, model, device_ids=None, output_device=None, broadcast_buffers=True,
                 find_unused_parameters=False, gradient_as_bucket_view=False, bucket_cap_mb=None,
                 grad_scaler=None, gradient_dtype=None, overlap_optimizer=None):
        super().__init__()
        if not pg.is_initialized():
            raise RuntimeError("Process group not initialized. Call genesis.distributed.init_process_group() first")
        object.__setattr__(self, "module", model)
        self.world_size = pg.get_world_size()
        self.rank = pg.get_rank()
        if device_ids is None:
            device_ids = [torch.cuda.current_device()] if torch.cuda.is_available() and pg._backend == "nccl" else None
        self.device_ids = device_ids
        self.output_device = output_device if output_device is not None else (device_ids[0] if device_ids else None)
        self.broadcast_buffers = broadcast_buffers
        self.find_unused_parameters = find_unused_parameters
        self.bucket_cap_bytes = int(float(bucket_cap_mb if bucket_cap_mb is not None
                                          else os.environ.get("GENESIS_DDP_BUCKET_MB", 100)) * 1024 * 1024)
        # The bucket that completes last (with tied embeddings: the embedding / output matrix, whose gradient is final
        # only when backward ends) is still being reduced when the optimizer starts.  With `overlap_optimizer` the
        # end of backward waits for every bucket but that one, tags its parameters with a join callback, and
        # `Optimizer.step` updates all other parameters first, joins, then updates the tagged ones: the tail of the
        # communication hides behind the optimizer kernel.  Anything else that reads those gradients first must call
        # `join_gradients()` (`clip_grad_norm_` does).  Off with a GradScaler: its overflow flag is complete only when
        # the last bucket is.  Default: on (GENESIS_DDP_OVERLAP_OPT=0 turns it off).
        self._overlap_opt = bool(int(os.environ.get("GENESIS_DDP_OVERLAP_OPT", "1"))) if overlap_optimizer is None \
            else bool(overlap_optimizer)
        self._early_done = None
        self._late_params = []
        self._sync = True
        self._scaler = grad_scaler
        # 16-bit wire format (`gradient_dtype="bfloat16"` / "float16", or GENESIS_DDP_GRAD_DTYPE): gradients stay
        # float32 in local buckets; the all-reduce kernel packs them to 16 bits, moves half the bytes over NVLink,
        # accumulates in float32 and casts the result back into the float32 bucket (both casts are phases of the
        # kernel).  Needs the peer-memory transport and float32 parameters.
        gd = gradient_dtype if gradient_dtype is not None else os.environ.get("GENESIS_DDP_GRAD_DTYPE") or None
        if gd is not None:
            from ..dtypes import get_dtype
            gd = get_dtype(gd).torch_dtype
            if gd == torch.float32:
                gd = None
            elif gd not in (torch.bfloat16, torch.float16):
                raise ValueError("gradient_dtype must be float32, bfloat16 or float16")
        self._wire_dtype = gd
        self._buckets = []
        self._param_bucket = {}
        self._next_launch = 0
        self._armed = False
        self._comm_stream = None
        self._use_symm = False
        self._probe = None
        # Wait budget of the bucket all-reduce.  Ranks legitimately drift apart by whole seconds between two steps
        # (rank 0 writing a checkpoint or running an evaluation while the others have already launched backward),
        # so the budget is far longer than that of the blocking collectives; NCCL would wait without any limit.
        self._budget_ms = float(os.environ.get("GENESIS_DDP_TIMEOUT_MS", 120000))
        # measurement switches: "skip" launches no all-reduce at all (compute time of the data-parallel layout; the
        # ranks diverge), "serial" reduces every bucket after backward (compute + communication with no overlap)
        self._debug_comm = os.environ.get("GENESIS_DDP_DEBUG_COMM", "")
        all_params = [p for p in model.parameters() if p.requires_grad]
        # expert-parallel shards are not replicated: no all-reduce, only the 1/world factor
        self._sharded = [p for p in all_params if getattr(p, "_no_ddp", False)]
        params = [p for p in all_params if not getattr(p, "_no_ddp", False)]
        self._on_cuda = bool(params) and params[0]._t.is_cuda
        if self.world_size > 1:
            self._broadcast_initial(model)
            self._build_buckets(params)
            for p in params:
                p.register_post_accumulate_grad_hook(self._make_hook())
        print(f"DDP: Initialized model on rank {self.rank}/{self.world_size}")

    # `.model` is the reference's second name for the wrapped module
    @property
    def model(self):
        return self.module

    # ---- construction ---------------------------------------------------------------
    def _broadcast_initial(self, model):
        tensors = [p._t for p in model.parameters() if not getattr(p, "_no_ddp", False)]
        if self.broadcast_buffers:
            tensors += [b._t for _, b in model.named_buffers()]
        # one flat broadcast per dtype instead of one per tensor
        by_dtype = {}
        for t in tensors:
            by_dtype.setdefault(t.dtype, []).append(t)
        for dt, ts in by_dtype.items():
            flat = torch.cat([t.reshape(-1) for t in ts])
            tdist.broadcast(flat, src=0)
            off = 0
            for t in ts:
                n = t.numel()
                t.copy_(flat[off:off + n].reshape(t.shape))
                off += n
        for p in model.parameters():
            p._version += 1            # overwritten in place: cached casts and low-precision copies are stale

    def _bucket_order(self, params):
        """Parameters in the order they get bucket slots: reverse registration order (roughly the order gradients
        become ready), except that parameters some layer multiplies as one stacked matrix (q/k/v, gate/up) sit next
        to each other in stacking order, so the fused weight-gradient GEMM can write all of them with one store
        straight into the bucket.  Returns a list of units (lists of parameters that must share a bucket)."""
        from .utils import fused_parameter_groups
        ids = {id(p) for p in params}
        group_of = {}
        for members in fused_parameter_groups(self.module):
            if all(id(m) in ids for m in members) and not any(id(m) in group_of for m in members) \
                    and len({m._t.dtype for m in members}) == 1:
                for m in members:
                    group_of[id(m)] = members
        units, done = [], set()
        for p in reversed(params):
            if id(p) in done:
                continue
            unit = list(group_of.get(id(p), [p]))
            done.update(id(m) for m in unit)
            units.append(unit)
        return units

    def _build_buckets(self, params):
        cur = {}
        for unit in self._bucket_order(params):
            unit_bytes = sum(m._t.numel() * m._t.element_size() for m in unit)
            for j, p in enumerate(unit):
                dt = p._t.dtype
                b = cur.get(dt)
                # a unit is never split across buckets: only its first member may open a new one
                if b is None or (j == 0 and b.numel > 0
                                 and b.numel * p._t.element_size() + unit_bytes > self.bucket_cap_bytes):
                    b = _Bucket(len(self._buckets), dt)
                    self._buckets.append(b)
                    cur[dt] = b
                # 16-byte aligned slots so vector loads never straddle parameters
                align = 16 // p._t.element_size()
                b.numel = (b.numel + align - 1) // align * align
                b.offsets.append(b.numel)
                b.params.append(p)
                b.numel += p._t.numel()
                self._param_bucket[id(p)] = b
        self._use_symm = self._on_cuda and comm_mode() == "p2p" and symm.available()
        if self._on_cuda:
            self._comm_stream = torch.cuda.Stream()
        if self._use_symm:
            # flag page of the communication stream (collective allocation: do it here); epochs counted on the
            # device so that a captured training step can be replayed
            symm.channel("ddp").use_device_epochs()
        if self._wire_dtype is not None and not self._use_symm:
            self._wire_dtype = None                     # NCCL / gloo transport: gradients stay in the parameter dtype
        for b in self._buckets:
            esz = torch.empty(0, dtype=b.dtype).element_size()
            pad = (b.numel + 1023) // 1024 * 1024          # slices stay 16-byte aligned for any world size <= 64
            wire = self._wire_dtype if b.dtype == torch.float32 else None
            if wire is not None:
                b.wire_dtype = wire
                b.symm_buf = symm.alloc(pad * 2)
                b.wire = b.symm_buf.view(wire, 0, pad)
                b.flat = torch.zeros(pad, dtype=b.dtype, device=b.params[0]._t.device)
            elif self._use_symm:
                b.symm_buf = symm.alloc(pad * esz)
                b.flat = b.symm_buf.view(b.dtype, 0, pad)
            else:
                b.flat = torch.zeros(pad, dtype=b.dtype, device=b.params[0]._t.device)
            for p, off in zip(b.params, b.offsets):
                p._grad_buf = b.flat[off:off + p._t.numel()].view(p._t.shape)
            b.pending = len(b.params)

    # ---- backward-time machinery ------------------------------------------------------
    def _make_hook(self):
        def hook(p):
            if not self._sync or not self._armed:
                return
            b = self._param_bucket[id(p)]
            b.pending -= 1
            if b.pending == 0:
                if self._on_cuda:
                    b.ready_event = torch.cuda.Event()
                    b.ready_event.record()
                self._launch_ready()
        return hook

    def _launch_ready(self):
        if self._debug_comm == "serial":
            return                            # every bucket is reduced at the end of backward (no overlap)
        while self._next_launch < len(self._buckets):
            b = self._buckets[self._next_launch]
            if b.pending != 0:
                break
            self._reduce_bucket(b)
            self._next_launch += 1

    def _reduce_bucket(self, b):
        b.launched = True
        scaler = self._scaler
        if self._debug_comm == "skip":
            return
        if self._on_cuda:
            st = self._comm_stream
            if self._tail_overlap() and b is self._buckets[-1]:
                self._early_done = torch.cuda.Event()
                self._early_done.record(st)          # every earlier bucket has been reduced at this point
            if b.ready_event is not None:
                st.wait_event(b.ready_event)
            else:
                st.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(st):
                if self._use_symm:
                    from ..ops import native as N
                    inv = found = None
                    if scaler is not None and scaler.is_enabled():
                        scaler._lazy_init(b.flat.device)
                        inv, found = scaler._scale, scaler._found_inf
                    if b.wire is not None:
                        N.allreduce_wire(symm.channel("ddp"), b.symm_buf, b.wire.numel(), b.wire_dtype, b.flat,
                                         inv_scale=inv, found_inf=found, prescale=1.0 / self.world_size,
                                         scale_is_reciprocal=True, budget_ms=self._budget_ms)
                    else:
                        N.allreduce_fused(symm.channel("ddp"), b.symm_buf, 0, b.flat.numel(), b.dtype, b.flat,
                                          inv_scale=inv, found_inf=found, prescale=1.0 / self.world_size,
                                          scale_is_reciprocal=True, budget_ms=self._budget_ms)
                else:
                    tdist.all_reduce(b.flat)
                    b.flat.mul_(1.0 / self.world_size)
        else:
            tdist.all_reduce(b.flat)
            b.flat.mul_(1.0 / self.world_size)

    def _finish_backward(self):
        """End of backward: flush buckets whose parameters got no gradient, join the comm stream."""
        if not self._armed:
            return
        self._armed = False
        if not self._sync:
            return
        for b in self._buckets[self._next_launch:]:
            # parameters without a gradient this step contribute zeros
            for p in b.params:
                if p.grad is None:
                    p._grad_buf.zero_()
                    if not self.find_unused_parameters:
                        p.grad = Tensor._wrap(p._grad_buf)
            b.pending = 0
            b.ready_event = None
            self._reduce_bucket(b)
        self._next_launch = len(self._buckets)
        fused_unscale = self._use_symm and self._scaler is not None and self._scaler.is_enabled()
        if self._sharded:
            from ..ops import dispatch as K
            grads = [p.grad._t for p in self._sharded if p.grad is not None]
            if grads and fused_unscale:
                # expert shards skip the all-reduce, and with it the unscale and the overflow check it carries:
                # do both here (1/world folded into the factor) so that every gradient reaches step() unscaled
                sc = self._scaler
                sc._lazy_init(grads[0].device)
                K.unscale_and_check(grads, (1.0 / self.world_size) / sc._scale, sc._found_inf)
            else:
                for g in grads:
                    K.mul_(g, 1.0 / self.world_size)
        if self._on_cuda and self._debug_comm != "skip":     # (nothing was launched on the stream when skipping)
            if self._early_done is not None:
                torch.cuda.current_stream().wait_event(self._early_done)
                self._early_done = None
                self._late_params = list(self._buckets[-1].params)
                for p in self._late_params:
                    p._late_join = self.join_gradients
            else:
                torch.cuda.current_stream().wait_stream(self._comm_stream)
        if fused_unscale:
            self._scaler._external_unscale = True
        if self._use_symm:
            # an all-reduce that gave up waiting leaves a record in the status word: fetch it without a host
            # synchronisation and look at it when the next forward starts (`Tensor.item()` looks at once)
            if self._probe is None:
                from ..ops import native as N
                self._probe = N.StatusProbe(self._buckets[0].flat.device) if self._buckets else None
            if self._probe is not None:
                self._probe.arm()

    def _tail_overlap(self):
        return self._overlap_opt and self._use_symm and not self._debug_comm and len(self._buckets) > 1 \
            and (self._scaler is None or not self._scaler.is_enabled())

    def join_gradients(self):
        """Make the current stream wait for the bucket all-reduce that `overlap_optimizer` left in flight at the end
        of backward.  Idempotent; called by `Optimizer.step`, `clip_grad_norm_` and the next forward."""
        if self._late_params:
            torch.cuda.current_stream().wait_stream(self._comm_stream)
            for p in self._late_params:
                p._late_join = None
            self._late_params = []

    def check_comm(self, wait=False):
        """Raise `CommTimeout` if a bucket all-reduce of an earlier step gave up waiting for a peer (its buckets
        then hold unreduced gradients).  Non-blocking unless `wait`; called by `forward` on every step."""
        if self._probe is not None:
            self._probe.poll("DistributedDataParallel gradient all-reduce", wait=wait)

    def _arm(self):
        self.join_gradients()
        self.check_comm()
        self._armed = True
        self._next_launch = 0
        self._early_done = None
        for b in self._buckets:
            b.pending = len(b.params)
            b.launched = False
            b.ready_event = None
        if self._finish_backward not in _backward_end_callbacks:
            _backward_end_callbacks.append(self._finish_backward)

    @contextlib.contextmanager
    def no_sync(self):
        """Skip gradient synchronisation inside the block (gradient accumulation)."""
        prev = self._sync
        self._sync = False
        try:
            yield
        finally:
            self._sync = prev

    def set_grad_scaler(self, scaler):
        self._scaler = scaler

    # ---- Module surface -----------------------------------------------------------------
    def forward(self, *inputs, **kwargs):
        if self.device_ids and self._on_cuda:
            dev = f"cuda:{self.device_ids[0]}"
            inputs = tuple(x.to(dev) if isinstance(x, Tensor) and not x._t.is_cuda else x for x in inputs)
            kwargs = {k: (v.to(dev) if isinstance(v, Tensor) and not v._t.is_cuda else v) for k, v in kwargs.items()}
        if self.world_size > 1:
            from .. import grad_mode
            if grad_mode.is_grad_enabled():
                self._arm()
        return self.module(*inputs, **kwargs)

    def state_dict(self, *a, **k):
        return self.module.state_dict(*a, **k)

    def load_state_dict(self, *a, **k):
        return self.module.load_state_dict(*a, **k)

    def parameters(self):
        return self.module.parameters()

    def named_parameters(self, *a, **k):
        return self.module.named_parameters(*a, **k)

    def buffers(self):
        return self.module.buffers()

    def named_buffers(self, *a, **k):
        return self.module.named_buffers(*a, **k)

    def modules(self):
        return self.module.modules()

    def named_modules(self, *a, **k):
        return self.module.named_modules(*a, **k)

    def train(self, mode=True):
        self.module.train(mode)
        self.training = mode
        return self

    def eval(self):
        return self.train(False)

    def to(self, *a, **k):
        self.module.to(*a, **k)
        return self

    def cuda(self, *a, **k):
        self.module.cuda(*a, **k)
        return self

    def cpu(self):
        self.module.cpu()
        return self

    def zero_grad(self):
        self.module.zero_grad()

    def __getattr__(self, name):
        # only reached when normal lookup fails: fall through to the wrapped module
        mod = self.__dict__.get("module")
        if mod is not None and name != "module":
            return getattr(mod, name)
        raise AttributeError(name)


DDP = DistributedDataParallel
