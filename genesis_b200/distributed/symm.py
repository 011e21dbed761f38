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
        self.status = torch.zeros(8, dtype=torch.int32, device=self.device)
        self.staging = None

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
    st = state()
    st.epoch += 1
    return st.epoch


def check_status(what="collective"):
    """Raise `CommTimeout` if a kernel recorded a bounded-wait expiry (synchronises the stream)."""
    st = state()
    rec = st.status.tolist()
    if rec[0] != 0:
        st.status.zero_()
        raise pg.CommTimeout(f"{what}: device-side wait expired (code={rec[0]}, peer={rec[1]}, phase={rec[2]}, "
                             f"epoch={rec[3]})")


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
