"""Symmetric heap over NVLink: identical-layout device buffers mapped into every rank.

Each rank `cudaMalloc`s its part, exports a CUDA IPC handle, and maps all peers' parts
(handles travel through the process group's object all-gather); the resulting table of
peer pointers is what the communication kernels (`csrc/comm.cu`) load from and store to
directly — plain `ld/st.global` on peer-mapped addresses, flags with system-scope
release/acquire, every wait bounded.  A wait that runs out writes a status record and the
kernel returns; `check_status()` turns it into `CommTimeout` on the host.
No NCCL call is made on these paths.  The reference has no counterpart (NCCL internals).
"""
import ctypes
import os

import torch
import torch.distributed as tdist

from .. import _lib
from . import process_group as pg

_state = None   # _SymmState


class _CAI:
    """Minimal `__cuda_array_interface__` carrier so torch can view a raw device pointer."""

    def __init__(self, ptr, nbytes):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


def tensor_from_ptr(ptr, nbytes, dtype, device):
    t = torch.as_tensor(_CAI(ptr, nbytes), device=device)
    return t.view(dtype)


class SymmBuffer:
    """One symmetric allocation: `local` is this rank's tensor view, `ptrs` the per-rank addresses."""

    def __init__(self, nbytes, local_ptr, peer_ptrs, device):
        self.nbytes, self.local_ptr, self.peer_ptrs, self.device = nbytes, local_ptr, peer_ptrs, device
        self.bytes = tensor_from_ptr(local_ptr, nbytes, torch.uint8, device)
        W = len(peer_ptrs)
        self.ptr_table = (ctypes.c_void_p * W)(*peer_ptrs)

    def view(self, dtype, offset_bytes=0, numel=None):
        esz = torch.empty(0, dtype=dtype).element_size()
        n = (self.nbytes - offset_bytes) // esz if numel is None else numel
        return self.bytes[offset_bytes:offset_bytes + n * esz].view(dtype)


class _SymmState:
    def __init__(self):
        self.lib = _lib.get(required=True)
        self.rank, self.world = pg.get_rank(), pg.get_world_size()
        self.device = torch.device("cuda", torch.cuda.current_device())
        self.buffers = []
        self.opened = []
        self.epoch = 0
        self._bind()
        # flags: per-(channel, peer) 32-bit epoch counters; status: error record written by kernels
        self.flags = self.alloc(64 * 1024)
        # the status word is the library-wide one: whatever reads a result on the host (`Tensor.item()`,
        # `native.check_status`, DDP's probe) also sees an expired communication wait
        from ..ops import native
        self.status = native.status_tensor(self.device)
        self.staging = None
        self.channels = {}

    def next_epoch(self):
        self.epoch += 1
        return self.epoch

    def channel(self, name):
        """A flag page and epoch counter of its own (collective on first use).  Kernels that may run at the
        same time on different streams (the bucket all-reduce on DDP's communication stream, the collectives
        and expert-parallel kernels on the compute stream) must not share flag slots: with a shared page a
        slower kernel's older epoch could overwrite the newer one a peer is waiting for."""
        if name not in self.channels:
            self.channels[name] = _Channel(self, self.alloc(64 * 1024))
        return self.channels[name]

    def _bind(self):
        L = self.lib
        if getattr(L, "_symm_bound", False):
            return
        L.gb_symm_alloc.argtypes = [ctypes.c_size_t, ctypes.POINTER(ctypes.c_void_p)]
        L.gb_symm_free.argtypes = [ctypes.c_void_p]
        L.gb_ipc_get_handle.argtypes = [ctypes.c_void_p, ctypes.c_char_p]
        L.gb_ipc_open_handle.argtypes = [ctypes.c_char_p, ctypes.POINTER(ctypes.c_void_p)]
        L.gb_ipc_close_handle.argtypes = [ctypes.c_void_p]
        L._symm_bound = True

    def alloc(self, nbytes):
        """Collective: every rank must call with the same size in the same order."""
        nbytes = (int(nbytes) + 255) // 256 * 256
        p = ctypes.c_void_p()
        rc = self.lib.gb_symm_alloc(nbytes, ctypes.byref(p))
        if rc != 0:
            raise RuntimeError(f"symmetric allocation of {nbytes} bytes failed (cuda error {rc})")
        handle = ctypes.create_string_buffer(64)
        rc = self.lib.gb_ipc_get_handle(p, handle)
        if rc != 0:
            raise RuntimeError(f"cudaIpcGetMemHandle failed (cuda error {rc})")
        gathered = [None] * self.world
        tdist.all_gather_object(gathered, bytes(handle.raw))
        ptrs = []
        for r, h in enumerate(gathered):
            if r == self.rank:
                ptrs.append(p.value)
            else:
                q = ctypes.c_void_p()
                rc = self.lib.gb_ipc_open_handle(h, ctypes.byref(q))
                if rc != 0:
                    raise RuntimeError(f"cudaIpcOpenMemHandle for rank {r} failed (cuda error {rc})")
                self.opened.append(q.value)
                ptrs.append(q.value)
        buf = SymmBuffer(nbytes, p.value, ptrs, self.device)
        self.buffers.append(buf)
        tdist.barrier()
        return buf

    def close(self):
        torch.cuda.synchronize()
        for q in self.opened:
            self.lib.gb_ipc_close_handle(ctypes.c_void_p(q))
        self.opened = []
        try:
            tdist.barrier()
        except Exception:
            pass
        for b in self.buffers:
            self.lib.gb_symm_free(ctypes.c_void_p(b.local_ptr))
        self.buffers = []


class _Channel:
    """What the communication kernels need from the state, with private flags and epochs."""

    def __init__(self, st, flags):
        self.rank, self.world, self.device, self.status, self.flags = st.rank, st.world, st.device, st.status, flags
        self.epoch = 0
        self.epoch_dev = None

    def next_epoch(self):
        if self.epoch_dev is not None:
            raise RuntimeError("this channel counts its epochs on the device; host epochs cannot be mixed in")
        self.epoch += 1
        return self.epoch

    def use_device_epochs(self):
        """Count epochs in device memory (advanced by the kernels themselves) instead of passing them by value, so
        launches on this channel can be captured in a CUDA graph.  Every rank must switch at the same point."""
        if self.epoch_dev is None:
            if self.epoch != 0:
                raise RuntimeError("switch to device epochs before the channel's first collective")
            self.epoch_dev = torch.zeros(2, dtype=torch.int32, device=self.device)
        return self


def available():
    return (pg.is_initialized() and pg._world_size > 1 and pg._backend == "nccl"
            and torch.cuda.is_available() and _lib.available())


def state():
    global _state
    if _state is None:
        if not available():
            raise RuntimeError("symmetric heap needs an initialised multi-rank nccl process group")
        _state = _SymmState()
    return _state


def shutdown():
    global _state
    if _state is not None:
        try:
            _state.close()
        finally:
            _state = None


def alloc(nbytes):
    return state().alloc(nbytes)


def next_epoch():
    return state().next_epoch()


def channel(name):
    return state().channel(name)


def check_status(what="collective"):
    """Raise `CommTimeout` if a kernel recorded a bounded-wait expiry (synchronises the stream)."""
    from ..ops import native
    native.check_status(state().device, what)


def all_reduce_(t, scale=None):
    """In-place SUM all-reduce of a contiguous CUDA tensor through a symmetric staging buffer.
    Returns False when the peer-memory path is unavailable (caller falls back to NCCL)."""
    if not available():
        return False
    from ..ops import native as N
    st = state()
    nbytes = t.numel() * t.element_size()
    cap = int(os.environ.get("GENESIS_SYMM_STAGING_MB", 64)) * 1024 * 1024
    if st.staging is None:
        st.staging = st.alloc(cap)
    if nbytes > cap:
        return False
    stage = st.staging.view(t.dtype, 0, t.numel())
    stage.copy_(t.reshape(-1))
    # the kernel works on whole 16-byte vectors split evenly over the ranks: round the length up
    # (the tail of the staging buffer is reduced too and simply never copied back)
    quantum = st.world * (16 // t.element_size())
    n_pad = (t.numel() + quantum - 1) // quantum * quantum
    if n_pad * t.element_size() > cap:
        return False
    N.allreduce_fused(st, st.staging, 0, n_pad, t.dtype, stage, inv_scale=None, found_inf=None,
                      prescale=1.0 if scale is None else scale)
    t.reshape(-1).copy_(stage)
    return True


def _staging(nbytes):
    st = state()
    cap = int(os.environ.get("GENESIS_SYMM_STAGING_MB", 64)) * 1024 * 1024
    if st.staging is None:
        st.staging = st.alloc(cap)
    return st if nbytes <= cap else None


def _stage(st, tensors):
    """Copies contiguous tensors back to back (16-byte aligned starts) into the staging buffer; returns
    their byte offsets."""
    offs, pos = [], 0
    for t in tensors:
        nb = t.numel() * t.element_size()
        if nb:
            st.staging.bytes[pos:pos + nb].copy_(t.reshape(-1).view(torch.uint8))
        offs.append(pos)
        pos += (nb + 15) // 16 * 16
    return offs


def all_gather_(outs, t):
    """outs[r] <- rank r's `t` (same shape on every rank), through peer loads.  False: not available."""
    if not available() or not t.is_cuda or not t.is_contiguous():
        return False
    nb = t.numel() * t.element_size()
    st = _staging(nb)
    if st is None or any((not o.is_contiguous()) or o.numel() * o.element_size() != nb for o in outs):
        return False
    from ..ops import native as N
    _stage(st, [t])
    W = st.world
    flat = torch.empty(W * nb, dtype=torch.uint8, device=t.device)
    N.peer_pull(st, st.staging, [0] * W, [nb] * W, [r * nb for r in range(W)], flat)
    for r, o in enumerate(outs):
        o.reshape(-1).view(torch.uint8).copy_(flat[r * nb:(r + 1) * nb])
    return True


def broadcast_(t, src):
    if not available() or not t.is_cuda or not t.is_contiguous():
        return False
    nb = t.numel() * t.element_size()
    st = _staging(nb)
    if st is None:
        return False
    from ..ops import native as N
    W = st.world
    if st.rank == src:
        _stage(st, [t])
    send_len = [nb if (st.rank == src and d != src) else 0 for d in range(W)]
    N.peer_pull(st, st.staging, [0] * W, send_len, [0] * W, t)
    return True


def reduce_scatter_(out, ins):
    """out <- sum over ranks of their ins[my rank] (float tensors of equal size)."""
    if not available() or not out.is_cuda or not out.is_contiguous() or out.dtype not in (
            torch.float32, torch.float16, torch.bfloat16):
        return False
    n = out.numel()
    vec = 16 // out.element_size()
    n_pad = (n + vec - 1) // vec * vec
    W = state().world
    st = _staging(W * n_pad * out.element_size())
    if st is None or len(ins) != W or any(i.numel() != n or i.dtype != out.dtype for i in ins):
        return False
    from ..ops import native as N
    stage = st.staging.view(out.dtype, 0, W * n_pad).view(W, n_pad)
    for r, i in enumerate(ins):
        stage[r, :n].copy_(i.reshape(-1))
    res = out if n_pad == n else torch.empty(n_pad, dtype=out.dtype, device=out.device)
    N.peer_reduce_scatter(st, st.staging, res, n_pad)
    if res is not out:
        out.reshape(-1).copy_(res[:n])
    return True


def all_to_all_(out, inp, out_rows, in_rows):
    """Row-wise all-to-all of 2-D (or 1-D) contiguous tensors: `in_rows[d]` rows go to rank d, `out_rows[s]`
    rows arrive from rank s."""
    if not available() or not inp.is_cuda or not inp.is_contiguous() or not out.is_contiguous():
        return False
    row_b = (inp.numel() // inp.shape[0] if inp.shape[0] else 0) * inp.element_size()
    if inp.shape[0] == 0:
        row_b = (out.numel() // out.shape[0] if out.shape[0] else 0) * out.element_size()
    st = _staging(inp.numel() * inp.element_size())
    if st is None:
        # sizes differ between ranks here, so a silent fallback on one rank only would leave the others waiting
        raise RuntimeError("all-to-all send larger than the symmetric staging buffer: raise GENESIS_SYMM_STAGING_MB "
                           "(same value on every rank) or set GENESIS_COMM=nccl")
    from ..ops import native as N
    _stage(st, [inp])
    W = st.world
    send_off, pos = [], 0
    for d in range(W):
        send_off.append(pos * row_b)
        pos += in_rows[d]
    recv_off, pos = [], 0
    for s_ in range(W):
        recv_off.append(pos * row_b)
        pos += out_rows[s_]
    N.peer_pull(st, st.staging, send_off, [r * row_b for r in in_rows], recv_off, out)
    return True


def barrier_():
    if not available():
        return False
    from ..ops import native as N
    N.peer_barrier(state())
    return True
