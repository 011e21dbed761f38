"""ctypes bindings of `libgenesis_b200.so` (hand-written sm_100a kernels, sources in `csrc/`).

Every wrapper takes and returns `torch.Tensor`s, launches on torch's current CUDA stream and
returns `NotImplemented` for inputs the kernel family does not cover (float64 / integer math,
misaligned views, > 6-D strided copies ...), in which case `dispatch` uses the generic op.
On a machine with a GPU the library is mandatory: import fails loudly if it is missing.
"""
import ctypes
import math
import os

import torch

from .. import _lib

F32, F16, BF16 = torch.float32, torch.float16, torch.bfloat16
_DT = {F32: 0, F16: 1, BF16: 2, torch.float64: 3, torch.int32: 4, torch.int64: 5, torch.uint8: 6, torch.bool: 7}
_FLOATS = (F32, F16, BF16)

_BIN = {"add": 0, "sub": 1, "mul": 2, "div": 3, "max": 4, "min": 5, "rsub": 6, "rdiv": 7, "pow": 8, "rpow": 9}
_UN = {"neg": 0, "exp": 1, "log": 2, "sqrt": 3, "rsqrt": 4, "sin": 5, "cos": 6, "tanh": 7, "sigmoid": 8, "relu": 9,
       "abs": 10, "sign": 11, "silu": 12, "gelu": 13, "reciprocal": 14}
_CMP = {"eq": 0, "ne": 1, "lt": 2, "le": 3, "gt": 4, "ge": 5}
_RED = {"sum": 0, "mean": 0, "max": 1, "min": 2}

_C = {"p": ctypes.c_void_p, "i": ctypes.c_int, "l": ctypes.c_longlong, "f": ctypes.c_float,
      "u": ctypes.c_ulonglong, "I": ctypes.c_uint, "z": ctypes.c_size_t, "d": ctypes.c_double}

# name -> argument type codes (see _C); the trailing stream is a "p"
_SIGS = {
    "gb_binary": "ippplip", "gb_binary_scalar": "ipfplip", "gb_binary_strided": "ippppppip",
    "gb_unary": "ipplip", "gb_unary_bwd": "ippplip", "gb_clamp": "ppfflip", "gb_compare": "ippfiplip",
    "gb_where": "pppffiiplip", "gb_cast": "ppliip", "gb_fill": "plfip", "gb_axpy": "ppfliip",
    "gb_copy_strided": "ppipppip", "gb_transpose": "ppiiilllip",
    "gb_reduce_rows": "ippllfiip", "gb_reduce_mid": "ipplllifiip",
    "gb_rmsnorm_fwd": "pppplifiip", "gb_rmsnorm_bwd": "pppppplii" + "ip",
    "gb_add_rmsnorm_fwd": "pppppplifiip", "gb_add_rmsnorm_bwd": "ppppppplii" + "ip", "gb_layernorm_fwd": "pppppplifiip",
    "gb_layernorm_bwd": "pppppppp" + "liiip", "gb_norm_bwd_ctas": "l", "gb_rmsnorm_bwd_ctas": "lii",
    "gb_softmax_fwd_stream": "ppllii" + "pp", "gb_rmsnorm_fwd_stream": "pppplifii" + "pp", "gb_softmax_fwd": "ppllii" + "p", "gb_softmax_bwd": "pppllii" + "p",
    "gb_ce_fwd": "ppppllliip", "gb_ce_bwd": "ppppplll" + "iip",
    "gb_swiglu_fwd": "ppplip", "gb_swiglu_bwd": "ppppplip",
    "gb_swiglu_fwd2d": "ppliip", "gb_swiglu_bwd2d": "pppliip", "gb_rope": "pppppiiiiiillp", "gb_qkv_rope": "ppppppp" + "liiiiii" + "p",
    "gb_gather_rows": "pppllilpp", "gb_scatter_add_rows": "pppliiilpp",
    "gb_random": "pluuiffip", "gb_randint": "pluullp", "gb_dropout": "ppplfuuip",
    "gb_opt_chunk": "", "gb_adam_multi": "pilfffffffiipppp", "gb_adam_dyn_advance": "pddpp", "gb_copy_h2d_async": "pplp", "gb_sgd_multi": "pilfffp",
    "gb_grad_multi": "pilpfppip",
    "gb_router_fwd": "ppppp" + "liiiip", "gb_router_bwd": "pppppp" + "liiiip",
    "gb_moe_sort": "pppppp" + "liiilp", "gb_moe_combine": "pppp" + "liiip", "gb_moe_combine_bwd": "pppppp" + "liiip",
    "gb_gemm": "pppp" + "iiii" + "ll" + "i" + "lll" + "ii" + "iii" + "i" + "f" + "i" + "p" + "i" + "ii" + "p" + "i" + "p",
    "gb_gemm_pair": "ppppp" + "iii" + "ll" + "ii" + "ii" + "iii" + "i" + "f" + "ii" + "pp",
    "gb_allreduce_fused": "ppllii" + "I" + "f" + "p" + "i" + "p" + "ii" + "u" + "ppp",
    "gb_allreduce_wire": "pplpii" + "I" + "f" + "p" + "i" + "p" + "ii" + "u" + "ppp",
    "gb_wait_flag": "pIupp",
    "gb_peer_pull": "pppppp" + "ii" + "I" + "i" + "u" + "pp",
    "gb_peer_reduce_scatter": "ppp" + "lii" + "I" + "f" + "ii" + "u" + "pp",
    "gb_peer_barrier": "p" + "ii" + "I" + "u" + "pp",
    "gb_ep_layout": "p" + "iiiii" + "pppppp" + "p", "gb_ep_stage_rows": "ppp" + "li" + "p",
    "gb_ep_dispatch_pull": "pppp" + "pppp" + "ppp" + "iiiiii" + "I" + "ii" + "u" + "pp",
    "gb_ep_combine_pull": "ppp" + "ppppp" + "pp" + "iiiiiiii" + "I" + "ii" + "u" + "pp",
    "gb_sort_rows": "ppp" + "liiii" + "pp", "gb_argmax_rows": "pp" + "liii" + "p",
    "gb_bincount": "pippli" + "p", "gb_nonzero_count": "ppli" + "p", "gb_nonzero_write": "pppli" + "p",
    "gb_triu_tril": "ppl" + "iiiii" + "p", "gb_one_hot": "pip" + "lii" + "p", "gb_arange": "pl" + "dd" + "i" + "p",
    "gb_repeat_interleave": "pp" + "lll" + "ii" + "p",
    "gb_cat": "ppp" + "i" + "p" + "ll" + "i" + "p",
    "gb_gather_dim": "ppp" + "ii" + "ppp" + "l" + "ii" + "pp",
    "gb_scatter_dim": "ppp" + "d" + "ii" + "ii" + "pppp" + "l" + "ii" + "pp",
    "gb_index_get": "pp" + "ppp" + "i" + "pp",
    "gb_index_put": "pp" + "d" + "ii" + "ppp" + "i" + "pp",
    "gb_masked_fill": "pp" + "d" + "ll" + "i" + "p", "gb_fill_elems": "pldip",
}

_L = None
_sm_count = {}
_status = {}


def lib():
    global _L
    if _L is None:
        L = _lib.get(required=True)
        for name, sig in _SIGS.items():
            fn = getattr(L, name)
            fn.argtypes = [_C[c] for c in sig]
            fn.restype = ctypes.c_int
        _L = L
    return _L


available = _lib.available


def _st():
    return torch.cuda.current_stream().cuda_stream


launch_count = 0   # native launches since import (every wrapper call below launches >= 1 kernel)


def _chk(rc, what):
    global launch_count
    launch_count += 1
    if rc != 0:
        raise RuntimeError(f"{what} failed with code {rc}")


def _sms(dev):
    i = dev.index if dev.index is not None else torch.cuda.current_device()
    if i not in _sm_count:
        _sm_count[i] = torch.cuda.get_device_properties(i).multi_processor_count
    return _sm_count[i]


def status_tensor(dev):
    """Per-device int32[8] word where kernels record a bounded-wait expiry."""
    i = dev.index if dev.index is not None else torch.cuda.current_device()
    if i not in _status:
        _status[i] = torch.zeros(8, dtype=torch.int32, device=dev)
    return _status[i]


def check_status(dev=None, what="native kernel"):
    """Synchronising read of the status word shared by every kernel of the library (compute and communication);
    raises if a kernel gave up waiting (`CommTimeout` when the expired wait was on a peer's flag), skipped an
    out-of-range index, or was sent more expert-parallel rows than its receive buffer holds."""
    dev = dev or torch.device("cuda", torch.cuda.current_device())
    st = status_tensor(dev)
    rec = st.tolist()
    if rec[0] != 0:
        st.zero_()
        _raise_status(rec, what)


def _raise_status(rec, what="native kernel"):
    if rec[0] == 4:
        raise IndexError(f"index out of range in a native kernel (site={rec[1]}: 1 row gather / embedding lookup, "
                         f"2 row scatter-add, 3 gather along a dim, 4 scatter along a dim, 5 indexed read, "
                         f"6 indexed write; block={rec[2]}, index={rec[3]}); the access was skipped")
    if rec[0] == 3 and rec[1] == 900:
        raise RuntimeError(f"{what}: expert-parallel receive buffer too small: this rank was sent {rec[3]} "
                           f"(tile-padded) rows; raise GENESIS_EP_CAPACITY (multiple of the balanced share)")
    if rec[0] == 2:
        from ..distributed.process_group import CommTimeout
        raise CommTimeout(f"{what}: device-side wait on a peer expired (code={rec[0]}, peer={rec[1]}, "
                          f"block={rec[2]}, epoch={rec[3]}); a rank is late, stopped or gone")
    raise RuntimeError(f"{what}: device-side wait expired: code={rec[0]} site={rec[1]} block={rec[2]} extra={rec[3]}")


class StatusProbe:
    """Sync-free look at the status word: `arm()` enqueues a device-to-host copy into pinned memory on the current
    stream; `poll()` raises once that copy has landed and shows a record.  DistributedDataParallel arms it at the
    end of every backward pass and polls at the next forward, so an expired wait of a gradient all-reduce stops
    training one step later without adding a host synchronisation."""

    def __init__(self, dev):
        self.dev = dev
        self.host = torch.zeros(8, dtype=torch.int32).pin_memory()
        self.event = None

    def arm(self):
        if torch.cuda.is_current_stream_capturing():
            return
        self.host.copy_(status_tensor(self.dev), non_blocking=True)
        self.event = torch.cuda.Event()
        self.event.record()

    def poll(self, what="gradient all-reduce", wait=False):
        if self.event is None:
            return
        if wait:
            self.event.synchronize()
        elif not self.event.query():
            return
        self.event = None
        rec = self.host.tolist()
        if rec[0] != 0:
            status_tensor(self.dev).zero_()
            _raise_status(rec, what)


def _ok(t):
    return t.dtype in _FLOATS and t.is_contiguous() and t.data_ptr() % 16 == 0


# =============================== elementwise =====================================
def binary(name, a, b):
    op = _BIN.get(name)
    ta, tb = isinstance(a, torch.Tensor), isinstance(b, torch.Tensor)
    if ta and tb:
        if a.dtype != b.dtype or a.dtype not in _FLOATS:
            return NotImplemented
        if a.shape == b.shape and _ok(a) and _ok(b):
            out = torch.empty_like(a)
            _chk(lib().gb_binary(op, a.data_ptr(), b.data_ptr(), out.data_ptr(), a.numel(), _DT[a.dtype], _st()), name)
            return out
        try:
            shape = torch.broadcast_shapes(a.shape, b.shape)
        except RuntimeError:
            return NotImplemented
        if len(shape) > 4:
            return NotImplemented
        ae, be = a.expand(shape), b.expand(shape)
        pad = 4 - len(shape)
        sh = (ctypes.c_longlong * 4)(*([1] * pad + list(shape)))
        sa = (ctypes.c_longlong * 4)(*([0] * pad + list(ae.stride())))
        sb = (ctypes.c_longlong * 4)(*([0] * pad + list(be.stride())))
        out = torch.empty(shape, dtype=a.dtype, device=a.device)
        _chk(lib().gb_binary_strided(op, a.data_ptr(), b.data_ptr(), out.data_ptr(), sh, sa, sb, _DT[a.dtype], _st()),
             name)
        return out
    if not ta and not tb:
        return NotImplemented
    t, s, rev = (a, b, False) if ta else (b, a, True)
    if not _ok(t) or isinstance(s, (bool, complex)) or not isinstance(s, (int, float)):
        return NotImplemented
    if rev:
        op = {"add": 0, "mul": 2, "sub": 6, "div": 7, "max": 4, "min": 5}.get(name)
        if op is None:
            return NotImplemented
    out = torch.empty_like(t)
    _chk(lib().gb_binary_scalar(op, t.data_ptr(), float(s), out.data_ptr(), t.numel(), _DT[t.dtype], _st()), name)
    return out


def scalar_op(name, t, s):
    if not _ok(t):
        return NotImplemented
    out = torch.empty_like(t)
    _chk(lib().gb_binary_scalar(_BIN[name], t.data_ptr(), float(s), out.data_ptr(), t.numel(), _DT[t.dtype], _st()),
         name)
    return out


def add_(a, b, alpha=1.0):
    if not (isinstance(b, torch.Tensor) and a.shape == b.shape and _ok(a) and b.dtype in _FLOATS
            and b.is_contiguous()):
        return NotImplemented
    _chk(lib().gb_axpy(a.data_ptr(), b.data_ptr(), float(alpha), a.numel(), _DT[a.dtype], _DT[b.dtype], _st()), "axpy")
    return a


def mul_(a, b):
    if isinstance(b, torch.Tensor) or not _ok(a):
        return NotImplemented
    _chk(lib().gb_binary_scalar(2, a.data_ptr(), float(b), a.data_ptr(), a.numel(), _DT[a.dtype], _st()), "mul_")
    return a


def unary(name, t):
    if name not in _UN or not _ok(t):
        return NotImplemented
    out = torch.empty_like(t)
    _chk(lib().gb_unary(_UN[name], t.data_ptr(), out.data_ptr(), t.numel(), _DT[t.dtype], _st()), name)
    return out


def unary_bwd(name, g, t, y=None):
    if name not in _UN:
        return NotImplemented
    if name in ("exp", "sqrt", "tanh", "sigmoid"):
        t = y if y is not None else t
    if name == "neg":
        t = g
    if t is None or not _ok(g) or not _ok(t) or g.dtype != t.dtype or g.shape != t.shape:
        return NotImplemented
    out = torch.empty_like(g)
    _chk(lib().gb_unary_bwd(_UN[name], g.data_ptr(), t.data_ptr(), out.data_ptr(), g.numel(), _DT[g.dtype], _st()),
         name)
    return out


def clamp(t, lo, hi):
    if not _ok(t):
        return NotImplemented
    out = torch.empty_like(t)
    _chk(lib().gb_clamp(t.data_ptr(), out.data_ptr(), float("-inf") if lo is None else float(lo),
                        float("inf") if hi is None else float(hi), t.numel(), _DT[t.dtype], _st()), "clamp")
    return out


def compare(name, a, b):
    if not isinstance(a, torch.Tensor) or not _ok(a):
        return NotImplemented
    out = torch.empty(a.shape, dtype=torch.bool, device=a.device)
    if isinstance(b, torch.Tensor):
        if b.shape != a.shape or b.dtype != a.dtype or not _ok(b):
            return NotImplemented
        _chk(lib().gb_compare(_CMP[name], a.data_ptr(), b.data_ptr(), 0.0, 0, out.data_ptr(), a.numel(),
                              _DT[a.dtype], _st()), name)
    elif isinstance(b, (int, float)) and not isinstance(b, bool):
        _chk(lib().gb_compare(_CMP[name], a.data_ptr(), None, float(b), 1, out.data_ptr(), a.numel(),
                              _DT[a.dtype], _st()), name)
    else:
        return NotImplemented
    return out


def where(c, a, b):
    ta, tb = isinstance(a, torch.Tensor), isinstance(b, torch.Tensor)
    ref = a if ta else (b if tb else None)
    if ref is None or not _ok(ref) or c.dtype != torch.bool or c.shape != ref.shape or not c.is_contiguous():
        return NotImplemented
    for x in (a, b):
        if isinstance(x, torch.Tensor) and (x.shape != ref.shape or x.dtype != ref.dtype or not _ok(x)):
            return NotImplemented
    out = torch.empty_like(ref)
    _chk(lib().gb_where(c.data_ptr(), a.data_ptr() if ta else None, b.data_ptr() if tb else None,
                        0.0 if ta else float(a), 0.0 if tb else float(b), 0 if ta else 1, 0 if tb else 1,
                        out.data_ptr(), ref.numel(), _DT[ref.dtype], _st()), "where")
    return out


def cast(t, dtype):
    if t.dtype not in _FLOATS or dtype not in _FLOATS or not t.is_contiguous() or t.data_ptr() % 16:
        return NotImplemented
    out = torch.empty(t.shape, dtype=dtype, device=t.device)
    _chk(lib().gb_cast(t.data_ptr(), out.data_ptr(), t.numel(), _DT[t.dtype], _DT[dtype], _st()), "cast")
    return out


def fill_(t, value):
    if not _ok(t):
        # integers, bool, float64 and unaligned float tensors: the element-wise fill
        if t.is_contiguous() and t.dtype in _DT:
            _chk(lib().gb_fill_elems(t.data_ptr(), t.numel(), float(value), _DT[t.dtype], _st()), "fill_elems")
            return t
        return NotImplemented
    _chk(lib().gb_fill(t.data_ptr(), t.numel(), float(value), _DT[t.dtype], _st()), "fill")
    return t


def _strided_copy(src, dst):
    nd = src.dim()
    if nd > 6 or nd == 0:
        return False
    shape, sst, dst_st, es = list(src.shape), list(src.stride()), list(dst.stride()), src.element_size()
    if sst[-1] == 1 and dst_st[-1] == 1 and es < 8:
        # rows that are contiguous on both sides move in wider units (up to 8 bytes) when extents, strides and base
        # addresses allow: fewer, fatter elements for the index arithmetic of the strided kernel
        for f in (8 // es, 4 // es, 2 // es):
            wb = es * f
            if f > 1 and shape[-1] % f == 0 and src.data_ptr() % wb == 0 and dst.data_ptr() % wb == 0 \
                    and all(v % f == 0 for v in sst[:-1]) and all(v % f == 0 for v in dst_st[:-1]):
                shape[-1] //= f
                sst[:-1] = [v // f for v in sst[:-1]]
                dst_st[:-1] = [v // f for v in dst_st[:-1]]
                es = wb
                break
    sh = (ctypes.c_longlong * 6)(*shape)
    ss = (ctypes.c_longlong * 6)(*sst)
    ds = (ctypes.c_longlong * 6)(*dst_st)
    _chk(lib().gb_copy_strided(src.data_ptr(), dst.data_ptr(), nd, sh, ss, ds, es, _st()), "copy")
    return True


def contiguous(t):
    if t.numel() == 0 or t.element_size() not in (1, 2, 4, 8) or t.is_complex():
        return NotImplemented
    out = torch.empty(t.shape, dtype=t.dtype, device=t.device)
    # batched 2-D transpose (last two dims swapped in memory) goes through the smem-tiled kernel
    if t.dim() >= 2 and t.stride(-2) == 1 and t.element_size() in (2, 4, 8):
        R, Cc = t.shape[-2], t.shape[-1]
        lead = t.shape[:-2]
        tt = t.transpose(-1, -2)           # [.., C, R] view whose last dim is memory-contiguous
        batch = 1
        for s in lead:
            batch *= s
        flat, s_b = None, 0
        if len(lead) == 0:
            flat = tt
        else:
            try:
                flat = tt.view(batch, Cc, R)
                s_b = flat.stride(0)
            except RuntimeError:
                flat = None
        if flat is not None and batch <= 65535:
            # dst[b][r][c] = src_mem[b][c][r]: kernel writes dst[b][c'][r'] = src[b][r'][c'] with R'=C.. so swap roles
            _chk(lib().gb_transpose(flat.data_ptr(), out.data_ptr(), batch, Cc, R, s_b, flat.stride(-2),
                                    flat.stride(-1), t.element_size(), _st()), "transpose")
            return out
    if not _strided_copy(t, out):
        return NotImplemented
    return out


def transpose_into(dst, src):
    """dst [C, R] (contiguous) <- src [R, C] (contiguous) transposed, through the shared-memory tile kernel."""
    if src.dim() != 2 or dst.dim() != 2 or not src.is_contiguous() or not dst.is_contiguous() \
            or dst.shape[0] != src.shape[1] or dst.shape[1] != src.shape[0] or dst.dtype != src.dtype \
            or src.element_size() not in (2, 4, 8):
        return NotImplemented
    R, Cc = src.shape
    if R == 0 or Cc == 0:
        return dst
    _chk(lib().gb_transpose(src.data_ptr(), dst.data_ptr(), 1, R, Cc, 0, Cc, 1, src.element_size(), _st()),
         "transpose")
    return dst


def copy_(dst, src):
    if dst.shape != src.shape or dst.numel() == 0:
        return NotImplemented
    if dst.dtype == src.dtype:
        if dst.element_size() not in (1, 2, 4, 8) or dst.dim() > 6 or dst.dim() == 0 or dst.is_complex():
            return NotImplemented
        if dst.is_contiguous() and src.is_contiguous():
            n = dst.numel() * dst.element_size()
            es = 8 if (n % 8 == 0 and dst.data_ptr() % 8 == 0 and src.data_ptr() % 8 == 0) else dst.element_size()
            one = (ctypes.c_longlong * 6)(n // es)
            st1 = (ctypes.c_longlong * 6)(1)
            _chk(lib().gb_copy_strided(src.data_ptr(), dst.data_ptr(), 1, one, st1, st1, es, _st()), "copy")
            return dst
        return dst if _strided_copy(src, dst) else NotImplemented
    if dst.dtype in _FLOATS and src.dtype in _FLOATS and dst.is_contiguous() and src.is_contiguous() \
            and dst.data_ptr() % 16 == 0 and src.data_ptr() % 16 == 0:
        _chk(lib().gb_cast(src.data_ptr(), dst.data_ptr(), src.numel(), _DT[src.dtype], _DT[dst.dtype], _st()), "cast")
        return dst
    return NotImplemented


# ================================= reductions ====================================
def _reduce3(op, x, outer, red, inner, scale, out_dtype):
    """x contiguous, viewed as [outer, red, inner] -> [outer, inner]."""
    L = lib()
    out = torch.empty(outer * inner, dtype=out_dtype, device=x.device)
    if inner == 1:
        _chk(L.gb_reduce_rows(op, x.data_ptr(), out.data_ptr(), outer, red, scale, _DT[x.dtype], _DT[out_dtype], _st()),
             "reduce_rows")
        return out
    if outer > 65535:
        return None
    splits = 1
    if red >= 512:
        # the column kernel covers 32 x (16 bytes) columns per CTA; split the reduced extent until ~4 CTAs per SM exist
        vec = 16 // x.element_size()
        ctas = outer * (-(-inner // (32 * vec)))
        if ctas < 148 * 4:
            splits = int(min(64, max(1, red // 64), -(-148 * 4 // ctas)))
    if splits == 1:
        _chk(L.gb_reduce_mid(op, x.data_ptr(), out.data_ptr(), outer, red, inner, 1, scale, _DT[x.dtype],
                             _DT[out_dtype], _st()), "reduce_mid")
        return out
    part = torch.empty(splits * outer * inner, dtype=F32, device=x.device)
    _chk(L.gb_reduce_mid(op, x.data_ptr(), part.data_ptr(), outer, red, inner, splits, 1.0, _DT[x.dtype], 0, _st()),
         "reduce_mid")
    _chk(L.gb_reduce_mid(op, part.data_ptr(), out.data_ptr(), 1, splits, outer * inner, 1, scale, 0,
                         _DT[out_dtype], _st()), "reduce_mid2")
    return out


def reduce(name, t, dims, keepdim):
    if t.dtype not in _FLOATS or t.numel() == 0:
        return NotImplemented
    op = _RED[name]
    x = t if t.is_contiguous() else None
    if x is None:
        c = contiguous(t)
        if c is NotImplemented:
            return NotImplemented
        x = c
    shape = list(x.shape)
    nd = len(shape)
    if dims is None:
        n = x.numel()
        scale = 1.0 / n if name == "mean" else 1.0
        C = 8192
        if n <= 65536:
            out = _reduce3(op, x, 1, n, 1, scale, x.dtype)
        else:
            R = n // C
            parts = torch.empty(R + 1, dtype=F32, device=x.device)
            _chk(lib().gb_reduce_rows(op, x.data_ptr(), parts.data_ptr(), R, C, 1.0, _DT[x.dtype], 0, _st()), "reduce")
            tail = x.reshape(-1)[R * C:]
            if tail.numel():
                _chk(lib().gb_reduce_rows(op, tail.data_ptr(), parts[R:].data_ptr(), 1, tail.numel(), 1.0,
                                          _DT[x.dtype], 0, _st()), "reduce")
                out = _reduce3(op, parts, 1, R + 1, 1, scale, x.dtype)
            else:
                out = _reduce3(op, parts[:R], 1, R, 1, scale, x.dtype)
        return out.reshape([1] * nd) if keepdim else out.reshape(())
    dims = sorted(set(dims))
    if not dims:
        return t
    # collapse runs of adjacent dims; reduce runs from the back so earlier indices stay valid
    runs, cur = [], [dims[0]]
    for d in dims[1:]:
        if d == cur[-1] + 1:
            cur.append(d)
        else:
            runs.append(cur)
            cur = [d]
    runs.append(cur)
    cur_shape = shape[:]
    for run in reversed(runs):
        outer = math.prod(cur_shape[:run[0]])
        red = math.prod(cur_shape[run[0]:run[-1] + 1])
        inner = math.prod(cur_shape[run[-1] + 1:])
        scale = 1.0 / red if name == "mean" else 1.0
        r = _reduce3(op, x, outer, red, inner, scale, x.dtype)
        if r is None:
            return NotImplemented
        x = r
        for d in run:
            cur_shape[d] = 1
    if keepdim:
        return x.reshape(cur_shape)
    return x.reshape([s for i, s in enumerate(cur_shape) if i not in dims])


# ================================== GEMM =========================================
_GEMM_DT = {F32: 0, F16: 1, BF16: 2}


def _aligned(t, ld):
    es = t.element_size()
    return t.data_ptr() % 16 == 0 and (ld * es) % 16 == 0


def _operand(t, want_contract_last):
    """Classify a 2-D operand. Returns (tensor, mn_major, ld) with the tensor possibly re-laid-out.
    `want_contract_last`: the logical layout is [rows, contraction]."""
    r, c = t.shape
    if t.stride(1) == 1 and (t.stride(0) >= c or r == 1) and _aligned(t, t.stride(0) if r > 1 else c):
        return t, 0, (t.stride(0) if r > 1 else c)
    # MN-major operands go to the tensor cores as they are for 16-bit types; the tf32 path takes
    # K-major operands only, so float32 transposed views are repacked below.
    if t.dtype != F32 and t.stride(0) == 1 and (t.stride(1) >= r or c == 1) \
            and _aligned(t, t.stride(1) if c > 1 else r):
        return t, 1, (t.stride(1) if c > 1 else r)
    es = t.element_size()
    mult = 16 // es
    cp = (c + mult - 1) // mult * mult
    buf = torch.zeros(r, cp, dtype=t.dtype, device=t.device) if cp != c else \
        torch.empty(r, cp, dtype=t.dtype, device=t.device)
    if copy_(buf[:, :c], t) is NotImplemented:
        buf[:, :c].copy_(t)
    return buf[:, :c], 0, cp


plan_override = None     # (tile width, split-K factor) forced by tuning sweeps


def _plan(M, N, K, es, can_split, sms):
    """Tile width (256 / 128) and k-split policy of the persistent kernel.  Returns (bn, splits): splits == 1 plain,
    splits == -1 stream-K (every CTA takes an equal share of all tile x k-iteration units and adds its partial
    tiles into the fp32 output), chosen when whole tiles would leave more than a quarter of the SM-waves idle.
    (With a nearly full last wave the CTAs of a stream-K run drift apart in k and stop sharing operand panels in
    L2: measured 0.225 ms against 0.111 ms for 896 x 4864 x 16384, so that case stays on whole tiles.)"""
    k_iters = max(1, -(-K * es // 128))
    bn = 256 if N > 128 else 128
    tiles = -(-M // 128) * -(-N // bn)
    waves = -(-tiles // sms)
    eff = tiles / (waves * sms)
    if can_split and eff < 0.75 and tiles * k_iters >= 32:
        return bn, -1
    if not can_split and N > 128:
        # no way to split k: narrower tiles can still fill a ragged last wave
        t128 = -(-M // 128) * -(-N // 128)
        eff128 = t128 / (-(-t128 // sms) * sms)
        if eff128 * 0.8 > eff:
            return 128, 1
    return bn, 1


pair_mode = os.environ.get("GENESIS_GEMM_PAIR", "auto")     # "auto" | "0" (never) | "1" (whenever the kernel applies)


def _pair_width(M, N, K, sms, a_mn=0, b_mn=0):
    """256 when the CTA-pair kernel (256 x 256 tiles on SM pairs) is expected to beat the single-CTA kernel for this
    problem, else 0.  Measured on the model's shapes: the pair kernel wins by 2-9 % on K-major x K-major products with
    many tiles and a short contraction (the forward projections out of the hidden size, where operand traffic into
    the SMs bounds the 128 x 256 tile: +7 % at 16384 x 4864 x 896 and 16384 x 1152 x 896), loses on long contractions
    (-2 % at K = 4864, -4 % at 16384 x 2048 x 8192, -15 % at 16384 cubed, where the single-CTA kernel's grouped
    rasterisation keeps more of both operands in L2), on MN-major operands (data / weight gradients) and on very wide
    outputs (the vocabulary projection); narrower pair tiles never pay."""
    if pair_mode == "0":
        return 0
    if pair_mode == "1":
        return 256
    if a_mn or b_mn or M < 2048 or N < 768 or N > 32768 or K > 1536:
        return 0
    tiles = -(-M // 256) * -(-N // 256)
    return 256 if tiles >= 2 * (sms // 2) else 0


def gemm_pair(a2, a_mn, lda, b2, b_mn, ldb, M, N, K, out, bias, accumulate, alpha, bn):
    """Launch of the CTA-pair kernel on classified operands (see `_operand`).  Returns False when it does not apply."""
    if a2.element_size() != 2 or out.data_ptr() % 16 or (N * out.element_size()) % 16 or (K * 2) % 16:
        return False
    if accumulate and out.dtype != F32:
        return False
    if b_mn and bn == 192:
        bn = 256
    rc = lib().gb_gemm_pair(a2.data_ptr(), b2.data_ptr(), out.data_ptr(), None,
                            None if bias is None else bias.data_ptr(), M, N, K, lda, ldb, N, 0, a_mn, b_mn,
                            _GEMM_DT[a2.dtype], _GEMM_DT[out.dtype], 0 if bias is None else _GEMM_DT[bias.dtype],
                            1 if accumulate else 0, float(alpha), 0, bn, status_tensor(a2.device).data_ptr(), _st())
    _chk(rc, "gemm_pair")
    return True


def linear_swiglu(x, w, want_gu=True):
    """(gu, h): gu = x @ w^T with w the stacked [2 I, K] gate | up weight, h = silu(gu[:, :I]) * gu[:, I:], from ONE
    GEMM whose epilogue applies the activation (CTA-pair kernel, csrc/gemm2_sm100.cu).  `NotImplemented` when the
    shape does not fit (I a multiple of 128, 16-bit contiguous operands)."""
    if x.dtype not in (F16, BF16) or w.dtype != x.dtype or w.dim() != 2 or not w.is_contiguous() or pair_mode == "0":
        return NotImplemented
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    M, K = x2.shape
    I2 = w.shape[0]
    if I2 % 256 or (K * 2) % 16 or not x2.is_contiguous() or x2.data_ptr() % 16 or w.data_ptr() % 16 or M == 0:
        return NotImplemented
    I = I2 // 2
    gu = torch.empty(M, I2, dtype=x.dtype, device=x.device) if want_gu else None
    h = torch.empty(M, I, dtype=x.dtype, device=x.device)
    rc = lib().gb_gemm_pair(x2.data_ptr(), w.data_ptr(), None if gu is None else gu.data_ptr(), h.data_ptr(), None,
                            M, I, K, K, K, I2, I, 0, 0, _GEMM_DT[x.dtype], _GEMM_DT[x.dtype], 0, 0, 1.0, 1, 256,
                            status_tensor(x.device).data_ptr(), _st())
    _chk(rc, "gemm_pair(swiglu)")
    return (None if gu is None else gu.reshape(*lead, I2)), h.reshape(*lead, I)


def dgrad_swiglu_bwd(gy, wd_t, gu):
    """d(gate | up) [M, 2 I] of a SwiGLU MLP from the gradient `gy` [M, H] of the down projection's output, the
    [I, H] K-major twin `wd_t` of the down weight and gate | up `gu` [M, 2 I] of the forward pass: ONE GEMM
    (dh = gy @ wd_t^T) on CTA pairs whose epilogue applies the SwiGLU backward; dh is never stored."""
    if gy.dtype not in (F16, BF16) or wd_t.dtype != gy.dtype or gu.dtype != gy.dtype or pair_mode == "0":
        return NotImplemented
    lead = gy.shape[:-1]
    g2 = gy.reshape(-1, gy.shape[-1])
    u2 = gu.reshape(-1, gu.shape[-1])
    M, H = g2.shape
    I = wd_t.shape[0]
    if wd_t.dim() != 2 or wd_t.shape[1] != H or u2.shape != (M, 2 * I) or I % 64 or (H * 2) % 16 or M == 0 \
            or not (g2.is_contiguous() and wd_t.is_contiguous() and u2.is_contiguous()) \
            or g2.data_ptr() % 16 or wd_t.data_ptr() % 16 or u2.data_ptr() % 32:       # gate | up is read 32 bytes at a time
        return NotImplemented
    dgu = torch.empty(M, 2 * I, dtype=gy.dtype, device=gy.device)
    rc = lib().gb_gemm_pair(g2.data_ptr(), wd_t.data_ptr(), dgu.data_ptr(), u2.data_ptr(), None, M, I, H, H, H,
                            2 * I, 2 * I, 0, 0, _GEMM_DT[gy.dtype], _GEMM_DT[gy.dtype], 0, 0, 1.0, 2, 256,
                            status_tensor(gy.device).data_ptr(), _st())
    _chk(rc, "gemm_pair(swiglu_bwd)")
    return dgu.reshape(*lead, 2 * I)


def gemm(a, b_t, out_dtype=None, bias=None, accum=None, alpha=1.0, out=None):
    """D[M, N] = a[M, K] @ b_t[N, K]^T for 2-D operands in any of the supported layouts.
    `a` / `b_t` may be transposed views (stride(0) == 1); misaligned ones are repacked.
    `accum`: D is added into this tensor; `out`: D is written into this (contiguous [M, N]) tensor."""
    if a.dtype not in _GEMM_DT or a.dtype != b_t.dtype:
        return NotImplemented
    M, K = a.shape
    N = b_t.shape[0]
    out_dtype = out_dtype or a.dtype
    if out_dtype not in _GEMM_DT:
        return NotImplemented
    if accum is not None:
        out = accum
        if not out.is_contiguous():
            return NotImplemented
    elif out is not None:
        if not out.is_contiguous() or out.dtype != out_dtype or out.numel() != M * N:
            return NotImplemented
    else:
        out = torch.empty(M, N, dtype=out_dtype, device=a.device)
    if M == 0 or N == 0:
        return out
    if K == 0:
        if accum is None:
            out.zero_()
        return out
    a2, a_mn, lda = _operand(a, True)
    b2, b_mn, ldb = _operand(b_t, True)
    if bias is not None and (bias.dtype not in _GEMM_DT or not bias.is_contiguous()):
        return NotImplemented
    sms = _sms(a.device)
    bn, splits = _plan(M, N, K, a.element_size(), out.dtype == F32 and bias is None, sms)
    if plan_override is not None:
        bn, splits = plan_override
    elif splits == 1 and a.element_size() == 2:
        pbn = _pair_width(M, N, K, sms, a_mn, b_mn)
        if pbn and gemm_pair(a2, a_mn, lda, b2, b_mn, ldb, M, N, K, out, bias, accum is not None, alpha, pbn):
            return out
    if splits < 0 and (out.data_ptr() % 16 or (N * out.element_size()) % 16):
        splits = 1                     # the add path of the epilogue needs a 16-byte aligned output
    if splits != 1 and accum is None:
        out.zero_()
    rc = lib().gb_gemm(a2.data_ptr(), b2.data_ptr(), out.data_ptr(), None if bias is None else bias.data_ptr(),
                       M, N, K, 1, lda, ldb, N, 0, 0, 0, a_mn, b_mn, _GEMM_DT[a.dtype], _GEMM_DT[out.dtype],
                       0 if bias is None else _GEMM_DT[bias.dtype], 0 if accum is None else 1, float(alpha),
                       0, None, 0, splits, bn, status_tensor(a.device).data_ptr(), sms, _st())
    _chk(rc, "gemm")
    return out


def bgemm(a, b_t, out_dtype=None, b_is_kn=False):
    """Batched: a [B, M, K] times b_t [B, N, K] (K-major), or with `b_is_kn` times b [B, K, N] as stored (the
    tensor cores read it MN-major: no transpose copy; 16-bit types only) -> [B, M, N].  Contiguous operands."""
    Bn, M, K = a.shape
    N = b_t.shape[2] if b_is_kn else b_t.shape[1]
    es = a.element_size()
    if not (a.is_contiguous() and b_t.is_contiguous() and (K * es) % 16 == 0 and a.data_ptr() % 16 == 0
            and b_t.data_ptr() % 16 == 0):
        return NotImplemented
    if b_is_kn and (es != 2 or (N * es) % 16 != 0):
        return NotImplemented
    out = torch.empty(Bn, M, N, dtype=out_dtype or a.dtype, device=a.device)
    if out.numel() == 0:
        return out
    rc = lib().gb_gemm(a.data_ptr(), b_t.data_ptr(), out.data_ptr(), None, M, N, K, Bn, K, N if b_is_kn else K, N,
                       M * K, N * K, M * N, 0, 1 if b_is_kn else 0, _GEMM_DT[a.dtype], _GEMM_DT[out.dtype], 0, 0, 1.0,
                       0, None, 0, 1, 0, status_tensor(a.device).data_ptr(), _sms(a.device), _st())
    _chk(rc, "bgemm")
    return out


def matmul(a, b):
    if a.dtype not in _GEMM_DT or a.dtype != b.dtype or a.dim() == 0 or b.dim() == 0:
        return NotImplemented
    a1, b1 = a.dim() == 1, b.dim() == 1
    aa = a.unsqueeze(0) if a1 else a
    bb = b.unsqueeze(-1) if b1 else b
    if bb.dim() == 2:
        lead = aa.shape[:-1]
        a2 = aa.reshape(-1, aa.shape[-1])
        r = gemm(a2, bb.t())
        if r is NotImplemented:
            return NotImplemented
        out = r.reshape(*lead, bb.shape[-1])
    else:
        try:
            bshape = torch.broadcast_shapes(aa.shape[:-2], bb.shape[:-2])
        except RuntimeError:
            return NotImplemented
        ae = aa.expand(*bshape, *aa.shape[-2:]).reshape(-1, *aa.shape[-2:])
        be = bb.expand(*bshape, *bb.shape[-2:]).reshape(-1, *bb.shape[-2:])
        ae = ae if ae.is_contiguous() else ae.contiguous()
        if ae.element_size() == 2 and (ae.shape[-1] * 2) % 16 == 0 and (be.shape[-1] * 2) % 16 == 0:
            # b stays [batch, K, N]: read MN-major by the tensor cores, no transpose copy
            r = bgemm(ae, be if be.is_contiguous() else be.contiguous(), b_is_kn=True)
            if r is not NotImplemented:
                out = r.reshape(*bshape, aa.shape[-2], bb.shape[-1])
                if a1:
                    out = out.squeeze(-2)
                if b1:
                    out = out.squeeze(-1)
                return out
        bt = be.transpose(-1, -2)
        bt = bt if bt.is_contiguous() else bt.contiguous()
        K = ae.shape[-1]
        mult = 16 // ae.element_size()
        if K % mult:
            pad = mult - K % mult
            ae = torch.nn.functional.pad(ae, (0, pad))
            bt = torch.nn.functional.pad(bt, (0, pad))
        r = bgemm(ae, bt)
        if r is NotImplemented:
            return NotImplemented
        out = r.reshape(*bshape, aa.shape[-2], bb.shape[-1])
    if a1:
        out = out.squeeze(-2)
    if b1:
        out = out.squeeze(-1)
    return out


def linear(x, w, bias, out_dtype):
    if x.dtype != w.dtype or x.dtype not in _GEMM_DT or w.dim() != 2:
        return NotImplemented
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    r = gemm(x2, w, out_dtype=out_dtype, bias=bias)
    if r is NotImplemented:
        return NotImplemented
    return r.reshape(*lead, w.shape[0])


def linear_dgrad(gy, w):
    if gy.dtype != w.dtype or gy.dtype not in _GEMM_DT:
        return NotImplemented
    lead = gy.shape[:-1]
    g2 = gy.reshape(-1, gy.shape[-1])
    r = gemm(g2, w.t())        # w.t() is [K, N] with stride(0) == 1: an MN-major B operand
    if r is NotImplemented:
        return NotImplemented
    return r.reshape(*lead, w.shape[1])


def linear_wgrad(gy, x, out_dtype, accum, out=None):
    if gy.dtype != x.dtype or gy.dtype not in _GEMM_DT:
        return NotImplemented
    g2 = gy.reshape(-1, gy.shape[-1])
    x2 = x.reshape(-1, x.shape[-1])
    return gemm(g2.t(), x2.t(), out_dtype=out_dtype or gy.dtype, accum=accum, out=out)


# ============================ norms / softmax / loss =============================
def _norm_ok(x, cols):
    v = 4 if x.dtype == F32 else 8
    return x.dtype in _FLOATS and x.is_contiguous() and x.data_ptr() % 16 == 0 and cols % v == 0 \
        and cols // v <= 256 * 8


def _wdt(x, w):
    if w.dtype == F32 or w.dtype == x.dtype:
        return _DT[w.dtype]
    return None


def rmsnorm_fwd(x, w, eps):
    cols = x.shape[-1]
    if not _norm_ok(x, cols) or _wdt(x, w) is None or not w.is_contiguous():
        return NotImplemented
    rows = x.numel() // cols
    y = torch.empty_like(x)
    rstd = torch.empty(rows, dtype=F32, device=x.device)
    if 8192 <= cols * x.element_size() <= 65536 and rows >= 64:
        # wide rows: streamed through shared memory with the next row's copy in flight (csrc/row_stream.cuh)
        rc = lib().gb_rmsnorm_fwd_stream(x.data_ptr(), w.data_ptr(), y.data_ptr(), rstd.data_ptr(), rows, cols,
                                         float(eps), _DT[x.dtype], _wdt(x, w), status_tensor(x.device).data_ptr(), _st())
        if rc != -9:
            _chk(rc, "rmsnorm_fwd_stream")
            return y, rstd
    _chk(lib().gb_rmsnorm_fwd(x.data_ptr(), w.data_ptr(), y.data_ptr(), rstd.data_ptr(), rows, cols, float(eps),
                              _DT[x.dtype], _wdt(x, w), _st()), "rmsnorm_fwd")
    return y, rstd


def add_rmsnorm_fwd(x, res, w, eps):
    """(s = x + res, rmsnorm(s) * w, rstd) in one pass over the rows."""
    cols = x.shape[-1]
    if not _norm_ok(x, cols) or not _norm_ok(res, cols) or res.dtype != x.dtype or res.shape != x.shape \
            or _wdt(x, w) is None or not w.is_contiguous():
        return NotImplemented
    rows = x.numel() // cols
    s, y = torch.empty_like(x), torch.empty_like(x)
    rstd = torch.empty(rows, dtype=F32, device=x.device)
    _chk(lib().gb_add_rmsnorm_fwd(x.data_ptr(), res.data_ptr(), s.data_ptr(), w.data_ptr(), y.data_ptr(),
                                  rstd.data_ptr(), rows, cols, float(eps), _DT[x.dtype], _wdt(x, w), _st()),
         "add_rmsnorm_fwd")
    return s, y, rstd


def add_rmsnorm_bwd(g, gres, x, w, rstd):
    """(rmsnorm_backward(g) + gres, dw): the gradient of either addend of the sum that was normalised."""
    cols = x.shape[-1]
    if not _norm_ok(x, cols) or not _norm_ok(g, cols) or not _norm_ok(gres, cols) or g.dtype != x.dtype \
            or gres.dtype != x.dtype or _wdt(x, w) is None:
        return NotImplemented
    rows = x.numel() // cols
    L = lib()
    nct = L.gb_rmsnorm_bwd_ctas(rows, cols, _DT[x.dtype])
    dx = torch.empty_like(x)
    part = torch.empty(nct * cols, dtype=F32, device=x.device)
    _chk(L.gb_add_rmsnorm_bwd(g.data_ptr(), gres.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(),
                              dx.data_ptr(), part.data_ptr(), rows, cols, _DT[x.dtype], _wdt(x, w), _st()),
         "add_rmsnorm_bwd")
    return dx, _colsum(part, nct, cols)


def _colsum(partial, nrows, cols):
    return _reduce3(0, partial, 1, nrows, cols, 1.0, F32)


def rmsnorm_bwd(g, x, w, rstd):
    cols = x.shape[-1]
    if not _norm_ok(x, cols) or not _norm_ok(g, cols) or g.dtype != x.dtype or _wdt(x, w) is None:
        return NotImplemented
    rows = x.numel() // cols
    L = lib()
    nct = L.gb_rmsnorm_bwd_ctas(rows, cols, _DT[x.dtype])
    dx = torch.empty_like(x)
    part = torch.empty(nct * cols, dtype=F32, device=x.device)
    _chk(L.gb_rmsnorm_bwd(g.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dx.data_ptr(), part.data_ptr(),
                          rows, cols, _DT[x.dtype], _wdt(x, w), _st()), "rmsnorm_bwd")
    return dx, _colsum(part, nct, cols)


def layernorm_fwd(x, w, b, eps):
    cols = x.shape[-1]
    if not _norm_ok(x, cols):
        return NotImplemented
    ref = w if w is not None else b
    wdt = _DT[x.dtype] if ref is None else _wdt(x, ref)
    if wdt is None or (w is not None and b is not None and w.dtype != b.dtype):
        return NotImplemented
    rows = x.numel() // cols
    y = torch.empty_like(x)
    mean = torch.empty(rows, dtype=F32, device=x.device)
    rstd = torch.empty(rows, dtype=F32, device=x.device)
    _chk(lib().gb_layernorm_fwd(x.data_ptr(), None if w is None else w.data_ptr(), None if b is None else b.data_ptr(),
                                y.data_ptr(), mean.data_ptr(), rstd.data_ptr(), rows, cols, float(eps),
                                _DT[x.dtype], wdt, _st()), "layernorm_fwd")
    return y, mean, rstd


def layernorm_bwd(g, x, w, mean, rstd):
    cols = x.shape[-1]
    if not _norm_ok(x, cols) or not _norm_ok(g, cols) or g.dtype != x.dtype:
        return NotImplemented
    wdt = _DT[x.dtype] if w is None else _wdt(x, w)
    if wdt is None:
        return NotImplemented
    rows = x.numel() // cols
    L = lib()
    nct = L.gb_norm_bwd_ctas(rows)
    dx = torch.empty_like(x)
    pw = torch.empty(nct * cols, dtype=F32, device=x.device)
    pb = torch.empty(nct * cols, dtype=F32, device=x.device)
    _chk(L.gb_layernorm_bwd(g.data_ptr(), x.data_ptr(), None if w is None else w.data_ptr(), mean.data_ptr(),
                            rstd.data_ptr(), dx.data_ptr(), pw.data_ptr(), pb.data_ptr(), rows, cols, _DT[x.dtype],
                            wdt, _st()), "layernorm_bwd")
    return dx, _colsum(pw, nct, cols), _colsum(pb, nct, cols)


def _to_last(x, dim):
    dim = dim % x.dim()
    if dim == x.dim() - 1:
        return x if x.is_contiguous() else None, False
    return None, True


def softmax_fwd(x, dim, log):
    if x.dtype not in _FLOATS or x.dim() == 0:
        return NotImplemented
    d = dim % x.dim()
    if d != x.dim() - 1:
        xt = x.transpose(d, -1)
        xc = contiguous(xt) if not xt.is_contiguous() else xt
        if xc is NotImplemented:
            return NotImplemented
        return softmax_fwd(xc, -1, log).transpose(d, -1)
    xc = x if x.is_contiguous() else contiguous(x)
    if xc is NotImplemented:
        return NotImplemented
    cols = xc.shape[-1]
    y = torch.empty_like(xc)
    rows = xc.numel() // cols
    if 8192 <= cols * xc.element_size() <= 65536 and rows >= 64:
        # wide rows: streamed through shared memory with the next row's copy in flight (csrc/row_stream.cuh)
        rc = lib().gb_softmax_fwd_stream(xc.data_ptr(), y.data_ptr(), rows, cols, 1 if log else 0, _DT[xc.dtype],
                                         status_tensor(xc.device).data_ptr(), _st())
        if rc != -9:
            _chk(rc, "softmax_fwd_stream")
            return y
    _chk(lib().gb_softmax_fwd(xc.data_ptr(), y.data_ptr(), rows, cols, 1 if log else 0, _DT[xc.dtype],
                              _st()), "softmax_fwd")
    return y


def softmax_bwd(g, y, dim, log):
    if g.dtype not in _FLOATS or g.dtype != y.dtype or g.dim() == 0:
        return NotImplemented
    d = dim % g.dim()
    if d != g.dim() - 1:
        gt, yt = g.transpose(d, -1), y.transpose(d, -1)
        gc = gt if gt.is_contiguous() else contiguous(gt)
        yc = yt if yt.is_contiguous() else contiguous(yt)
        if gc is NotImplemented or yc is NotImplemented:
            return NotImplemented
        return softmax_bwd(gc, yc, -1, log).transpose(d, -1)
    gc = g if g.is_contiguous() else contiguous(g)
    yc = y if y.is_contiguous() else contiguous(y)
    if gc is NotImplemented or yc is NotImplemented:
        return NotImplemented
    cols = gc.shape[-1]
    dx = torch.empty_like(gc)
    _chk(lib().gb_softmax_bwd(gc.data_ptr(), yc.data_ptr(), dx.data_ptr(), gc.numel() // cols, cols, 1 if log else 0,
                              _DT[gc.dtype], _st()), "softmax_bwd")
    return dx


def cross_entropy_fwd(logits, target, ignore_index):
    if logits.dtype not in _FLOATS or not logits.is_contiguous() or target.dtype not in (torch.int64, torch.int32) \
            or not target.is_contiguous():
        return NotImplemented
    rows, cols = logits.shape
    loss = torch.empty(rows, dtype=F32, device=logits.device)
    lse = torch.empty(rows, dtype=F32, device=logits.device)
    ii = -(2 ** 62) if ignore_index is None else int(ignore_index)
    _chk(lib().gb_ce_fwd(logits.data_ptr(), target.data_ptr(), loss.data_ptr(), lse.data_ptr(), rows, cols, ii,
                         _DT[logits.dtype], 1 if target.dtype == torch.int64 else 0, _st()), "ce_fwd")
    return loss, lse


def cross_entropy_bwd(logits, target, lse, grad_rows, ignore_index, inplace):
    if logits.dtype not in _FLOATS or not logits.is_contiguous() or grad_rows.dtype != F32 \
            or not grad_rows.is_contiguous():
        return NotImplemented
    rows, cols = logits.shape
    out = logits if inplace else torch.empty_like(logits)
    ii = -(2 ** 62) if ignore_index is None else int(ignore_index)
    _chk(lib().gb_ce_bwd(logits.data_ptr(), target.data_ptr(), lse.data_ptr(), grad_rows.data_ptr(), out.data_ptr(),
                         rows, cols, ii, _DT[logits.dtype], 1 if target.dtype == torch.int64 else 0, _st()), "ce_bwd")
    return out


# ============================== transformer pieces ===============================
def swiglu_fwd(gate, up):
    if not _ok(gate) or not _ok(up) or gate.dtype != up.dtype or gate.shape != up.shape:
        return NotImplemented
    out = torch.empty_like(gate)
    _chk(lib().gb_swiglu_fwd(gate.data_ptr(), up.data_ptr(), out.data_ptr(), gate.numel(), _DT[gate.dtype], _st()),
         "swiglu_fwd")
    return out


def swiglu_bwd(g, gate, up):
    if not (_ok(g) and _ok(gate) and _ok(up)) or not (g.dtype == gate.dtype == up.dtype):
        return NotImplemented
    dg, du = torch.empty_like(gate), torch.empty_like(up)
    _chk(lib().gb_swiglu_bwd(g.data_ptr(), gate.data_ptr(), up.data_ptr(), dg.data_ptr(), du.data_ptr(), g.numel(),
                             _DT[g.dtype], _st()), "swiglu_bwd")
    return dg, du


def swiglu_fused_fwd(gu):
    """gu [..., 2 I] = gate | up -> silu(gate) * up [..., I]."""
    I = gu.shape[-1] // 2
    v = 16 // gu.element_size()
    if gu.dtype not in _FLOATS or not gu.is_contiguous() or gu.shape[-1] % 2 or I % v or gu.data_ptr() % 16:
        return NotImplemented
    out = torch.empty(gu.shape[:-1] + (I,), dtype=gu.dtype, device=gu.device)
    _chk(lib().gb_swiglu_fwd2d(gu.data_ptr(), out.data_ptr(), gu.numel() // (2 * I), I, _DT[gu.dtype], _st()),
         "swiglu_fwd2d")
    return out


def swiglu_fused_bwd(dy, gu):
    I = gu.shape[-1] // 2
    v = 16 // gu.element_size()
    if gu.dtype not in _FLOATS or dy.dtype != gu.dtype or not gu.is_contiguous() or not dy.is_contiguous() \
            or I % v or gu.data_ptr() % 16 or dy.data_ptr() % 16:
        return NotImplemented
    dgu = torch.empty_like(gu)
    _chk(lib().gb_swiglu_bwd2d(dy.data_ptr(), gu.data_ptr(), dgu.data_ptr(), gu.numel() // (2 * I), I, _DT[gu.dtype],
                               _st()), "swiglu_bwd2d")
    return dgu


def _token_rows(t):
    """(row stride in elements, ok) of a [B, S, H, D] tensor whose last two dims are dense and whose (b, s) rows are
    equally spaced (a contiguous tensor, or a column slice of a wider [B, S, N] matrix)."""
    B, S, H, D = t.shape
    if t.stride(3) != 1 or (H > 1 and t.stride(2) != D):
        return 0, False
    rs = t.stride(1) if S > 1 else H * D
    if B > 1 and t.stride(0) != S * rs:
        return 0, False
    return rs, True


def rope(x, cos, sin, positions, inverse, out=None):
    """Rotate-half RoPE.  `x` and `out` may be column slices of wider matrices (equal token-row spacing)."""
    if x.dtype not in _FLOATS or x.dim() != 4 or cos.dtype != F32 or sin.dtype != F32 \
            or not cos.is_contiguous() or not sin.is_contiguous() or x.shape[-1] % 2:
        return NotImplemented
    xrs, ok = _token_rows(x)
    if not ok:
        return NotImplemented
    B, S, H, D = x.shape
    pos_ptr = None
    if positions is not None:
        positions = positions.to(torch.int64).contiguous()
        if positions.dim() == 1:
            positions = positions.unsqueeze(0).expand(B, S).contiguous()
        pos_ptr = positions.data_ptr()
    elif cos.shape[0] < S:
        return NotImplemented
    if out is None:
        out = torch.empty(B, S, H, D, dtype=x.dtype, device=x.device)
    ors, ok = _token_rows(out)
    if not ok or out.dtype != x.dtype or out.shape != x.shape:
        return NotImplemented
    _chk(lib().gb_rope(x.data_ptr(), out.data_ptr(), cos.data_ptr(), sin.data_ptr(), pos_ptr, B, S, H, D,
                       1 if inverse else 0, _DT[x.dtype], xrs, ors, _st()), "rope")
    return out


def qkv_rope(y, q, k, v, cos, sin, positions, Hq, Hkv, D, merge):
    """One launch over the three head groups of a fused projection: split (`merge=False`: y [B, S, (Hq + 2 Hkv) D] ->
    rotated q, rotated k, v, all freshly allocated when passed as None) or merge (`merge=True`: gradients q, k, v ->
    y, rotated back).  Returns (y, q, k, v) or NotImplemented."""
    t = y if y is not None else q
    if t.dtype not in _FLOATS or cos.dtype != F32 or sin.dtype != F32 or not cos.is_contiguous() \
            or not sin.is_contiguous():
        return NotImplemented
    B, S = t.shape[0], t.shape[1]
    Nt = (Hq + 2 * Hkv) * D
    dev, dt = t.device, t.dtype
    if merge:
        if any(g is None or g.dtype != dt or not g.is_contiguous() for g in (q, k, v)):
            return NotImplemented
        y = torch.empty(B, S, Nt, dtype=dt, device=dev)
    else:
        if not y.is_contiguous() or y.shape[-1] != Nt:
            return NotImplemented
        q = torch.empty(B, S, Hq, D, dtype=dt, device=dev)
        k = torch.empty(B, S, Hkv, D, dtype=dt, device=dev)
        v = torch.empty(B, S, Hkv, D, dtype=dt, device=dev)
    pos_ptr = None
    if positions is not None:
        positions = positions.to(torch.int64).contiguous()
        if positions.dim() == 1:
            positions = positions.unsqueeze(0).expand(B, S).contiguous()
        pos_ptr = positions.data_ptr()
    elif cos.shape[0] < S:
        return NotImplemented
    rc = lib().gb_qkv_rope(y.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), cos.data_ptr(), sin.data_ptr(),
                           pos_ptr, B * S, S, Hq, Hkv, D, 1 if merge else 0, _DT[dt], _st())
    if rc == -9:
        return NotImplemented
    _chk(rc, "qkv_rope")
    return y, q, k, v


def gather_rows(x, rows):
    if x.dim() != 2 or not x.is_contiguous() or rows.dtype not in (torch.int64, torch.int32) \
            or not rows.is_contiguous():
        return NotImplemented
    rb = x.shape[1] * x.element_size()
    if rb % 16 or x.data_ptr() % 16:
        return NotImplemented
    out = torch.empty(rows.numel(), x.shape[1], dtype=x.dtype, device=x.device)
    _chk(lib().gb_gather_rows(x.data_ptr(), rows.data_ptr(), out.data_ptr(), rows.numel(), rb,
                              1 if rows.dtype == torch.int64 else 0, x.shape[0], status_tensor(x.device).data_ptr(),
                              _st()), "gather_rows")
    return out


def embedding_fwd(weight, idx):
    if weight.dim() != 2:
        return NotImplemented
    flat = idx.reshape(-1)
    flat = flat if flat.is_contiguous() else flat.contiguous()
    r = gather_rows(weight, flat)
    if r is NotImplemented:
        return NotImplemented
    return r.reshape(*idx.shape, weight.shape[1])


def scatter_add_rows(src, rows, num_rows, out_dtype):
    if src.dtype not in _FLOATS or src.dim() != 2 or not src.is_contiguous() \
            or rows.dtype not in (torch.int64, torch.int32) or not rows.is_contiguous():
        return NotImplemented
    acc = torch.zeros(num_rows, src.shape[1], dtype=F32, device=src.device)
    _chk(lib().gb_scatter_add_rows(src.data_ptr(), rows.data_ptr(), acc.data_ptr(), src.shape[0], src.shape[1],
                                   _DT[src.dtype], 1 if rows.dtype == torch.int64 else 0, num_rows,
                                   status_tensor(src.device).data_ptr(), _st()), "scatter_add_rows")
    od = out_dtype or src.dtype
    return acc if od == F32 else cast(acc, od)


def scatter_add_rows_into(src, rows, acc):
    """acc[rows[i]] += src[i] in place (acc fp32 [num_rows, D] contiguous)."""
    if src.dtype not in _FLOATS or src.dim() != 2 or not src.is_contiguous() or acc.dtype != F32 \
            or not acc.is_contiguous() or acc.dim() != 2 or acc.shape[1] != src.shape[1] \
            or rows.dtype not in (torch.int64, torch.int32) or not rows.is_contiguous():
        return NotImplemented
    _chk(lib().gb_scatter_add_rows(src.data_ptr(), rows.data_ptr(), acc.data_ptr(), src.shape[0], src.shape[1],
                                   _DT[src.dtype], 1 if rows.dtype == torch.int64 else 0, acc.shape[0],
                                   status_tensor(src.device).data_ptr(), _st()), "scatter_add_rows")
    return True


def embedding_bwd(g, idx, num_rows, out_dtype):
    D = g.shape[-1]
    g2 = g.reshape(-1, D)
    g2 = g2 if g2.is_contiguous() else g2.contiguous()
    flat = idx.reshape(-1)
    flat = flat if flat.is_contiguous() else flat.contiguous()
    return scatter_add_rows(g2, flat, num_rows, out_dtype)


def dropout_fwd(x, p, seed, offset):
    if not _ok(x):
        return NotImplemented
    y = torch.empty_like(x)
    mask = torch.empty(x.shape, dtype=torch.uint8, device=x.device)
    _chk(lib().gb_dropout(x.data_ptr(), y.data_ptr(), mask.data_ptr(), x.numel(), float(p), int(seed), int(offset),
                          _DT[x.dtype], _st()), "dropout")
    return y, mask


def random_fill(kind, shape, dtype, dev, seed, offset, a, b):
    with torch.cuda.device(dev):
        if kind == "randint":
            out = torch.empty(shape, dtype=torch.int64, device=dev)
            _chk(lib().gb_randint(out.data_ptr(), out.numel(), int(seed), int(offset), int(a), int(b), _st()), "randint")
            return out if dtype == torch.int64 else out.to(dtype)
        if dtype not in _FLOATS:
            return NotImplemented
        out = torch.empty(shape, dtype=dtype, device=dev)
        _chk(lib().gb_random(out.data_ptr(), out.numel(), int(seed), int(offset), 0 if kind == "uniform" else 1,
                             float(a), float(b), _DT[dtype], _st()), "random")
        return out


# ================================== optimisers ===================================
# Host side of pointer tables uploaded while a CUDA graph is being captured: the captured copy node reads the host
# block again on every replay, so the block must stay alive and unchanged.  `begin_capture_arena` reserves pinned
# memory BEFORE the capture starts (no pinned allocation inside it); tables are carved out of it and never reused.
_capture_keepalive = []
_capture_arena = None
_capture_arena_used = 0


def begin_capture_arena(nwords=1 << 20):
    global _capture_arena, _capture_arena_used
    _capture_arena = torch.empty(nwords, dtype=torch.int64).pin_memory()
    _capture_keepalive.append(_capture_arena)
    _capture_arena_used = 0



def _meta(rows, nt, dev):
    """Upload the pointer table (rows x nt int64) through a pinned staging buffer."""
    # torch's pinned-host allocator keeps a staging block alive until the async copy that reads it
    # has completed, so a fresh pinned tensor per call is both safe and cheap (blocks are recycled).
    flat = torch.tensor(rows, dtype=torch.int64).reshape(-1)
    if torch.cuda.is_current_stream_capturing():
        global _capture_arena_used
        n = flat.numel()
        if _capture_arena is None or _capture_arena_used + n > _capture_arena.numel():
            raise RuntimeError("pointer-table upload inside a CUDA-graph capture without a reserved pinned arena: "
                               "capture through genesis_b200.cuda.graph / make_graphed_callable")
        host = _capture_arena[_capture_arena_used:_capture_arena_used + n]
        _capture_arena_used += n
        host.copy_(flat)
        out = torch.empty(n, dtype=torch.int64, device=dev)
        _chk(lib().gb_copy_h2d_async(out.data_ptr(), host.data_ptr(), n * 8, _st()), "copy_h2d_async")
        return out
    return flat.pin_memory().to(dev, non_blocking=True)


def _multi_table(params, grads, s1, s2, shadows):
    L = lib()
    chunk = L.gb_opt_chunk()
    nt = len(params)
    starts, total = [], 0
    for g in grads:
        starts.append(total)
        total += (g.numel() + chunk - 1) // chunk
    z = [0] * nt
    rows = [[p.data_ptr() for p in params] if params[0] is not None else z,
            [g.data_ptr() for g in grads],
            [t.data_ptr() for t in s1] if s1 is not None else z,
            [t.data_ptr() for t in s2] if s2 is not None else z,
            [0 if (shadows is None or s is None) else s.data_ptr() for s in (shadows or params)] if shadows else z,
            [g.numel() for g in grads], starts, [_DT[g.dtype] for g in grads]]
    return rows, nt, total


def _opt_ok(params, grads, states):
    for p, g in zip(params, grads):
        if p.dtype != F32 or not p.is_contiguous() or g.dtype not in _FLOATS or not g.is_contiguous() \
                or g.numel() != p.numel():
            return False
    for st in states:
        if st is not None:
            for t in st:
                if t.dtype != F32 or not t.is_contiguous():
                    return False
    return True


def adamw_step(params, grads, ms, vs, lr, beta1, beta2, eps, weight_decay, step, decoupled, grad_scale, found_inf,
               shadows, dyn=None, advance=True):
    """`dyn` (device fp32 [4]: lr, bias corrections, step count) moves the step-dependent scalars to the device:
    the kernel advances the count itself, so the launch sequence can be replayed from a CUDA graph."""
    if not _opt_ok(params, grads, (ms, vs)):
        return NotImplemented
    sdt = 0
    if shadows is not None:
        sd = {s.dtype for s in shadows if s is not None}
        if len(sd) > 1 or any(d not in _FLOATS for d in sd):
            return NotImplemented
        sdt = _DT[sd.pop()] if sd else 0
    rows, nt, total = _multi_table(params, grads, ms, vs, shadows)
    dev = params[0].device
    meta = _meta(rows, nt, dev)
    gs = None if grad_scale is None else grad_scale.data_ptr()
    fi = None if found_inf is None else found_inf.data_ptr()
    dp = None
    if dyn is not None:
        dp = dyn.data_ptr()
        if advance:
            _chk(lib().gb_adam_dyn_advance(dp, float(beta1), float(beta2), fi, _st()), "adam_dyn_advance")
    _chk(lib().gb_adam_multi(meta.data_ptr(), nt, total, float(lr), float(beta1), float(beta2), float(eps),
                             float(weight_decay), 1.0 - beta1 ** step, 1.0 - beta2 ** step, 1 if decoupled else 0,
                             sdt, gs, fi, dp, _st()), "adam_multi")
    return True


def sgd_step(params, grads, bufs, lr, momentum, weight_decay):
    if not _opt_ok(params, grads, (bufs,)):
        return NotImplemented
    rows, nt, total = _multi_table(params, grads, bufs, None, None)
    meta = _meta(rows, nt, params[0].device)
    _chk(lib().gb_sgd_multi(meta.data_ptr(), nt, total, float(lr), float(momentum), float(weight_decay), _st()),
         "sgd_multi")
    return True


def _grad_multi(grads, scale, found_inf, norm_sq, mode):
    for g in grads:
        if g.dtype not in _FLOATS or not g.is_contiguous():
            return NotImplemented
    rows, nt, total = _multi_table([None] * len(grads), grads, None, None, None)
    meta = _meta(rows, nt, grads[0].device)
    sp, fs = None, 1.0
    if isinstance(scale, torch.Tensor):
        sp = scale.data_ptr()
    elif scale is not None:
        fs = float(scale)
    _chk(lib().gb_grad_multi(meta.data_ptr(), nt, total, sp, fs, None if found_inf is None else found_inf.data_ptr(),
                             None if norm_sq is None else norm_sq.data_ptr(), mode, _st()), "grad_multi")
    return True


def unscale_and_check(grads, inv_scale, found_inf):
    if isinstance(inv_scale, torch.Tensor) and inv_scale.dtype != F32:
        return NotImplemented
    return _grad_multi(grads, inv_scale, found_inf, None, (1 if inv_scale is not None else 0) | 2)


def grad_norm_sq(grads, out):
    return _grad_multi(grads, None, None, out, 4)


# =================================== MoE =========================================
def moe_router(logits, k, renorm):
    if logits.dtype not in _FLOATS or logits.dim() != 2 or not logits.is_contiguous() or logits.shape[1] > 256 \
            or k > 32:
        return NotImplemented
    T, E = logits.shape
    dev = logits.device
    w = torch.empty(T, k, dtype=F32, device=dev)
    e = torch.empty(T, k, dtype=torch.int32, device=dev)
    probs = torch.empty(T, E, dtype=F32, device=dev)
    counts = torch.empty(E, dtype=torch.int32, device=dev)
    _chk(lib().gb_router_fwd(logits.data_ptr(), w.data_ptr(), e.data_ptr(), probs.data_ptr(), counts.data_ptr(), T, E,
                             k, 1 if renorm else 0, _DT[logits.dtype], _st()), "router_fwd")
    e._gb_counts = counts          # lets the sort reuse the histogram
    return w, e, probs, counts


def moe_router_bwd(dweights, dprobs, probs, experts, weights, renorm):
    if probs.dtype != F32 or experts.dtype != torch.int32:
        return NotImplemented
    T, E = probs.shape
    k = experts.shape[1]
    dw = None if dweights is None else dweights.to(F32).contiguous()
    dp = None if dprobs is None else dprobs.to(F32).contiguous()
    out = torch.empty(T, E, dtype=F32, device=probs.device)
    _chk(lib().gb_router_bwd(None if dw is None else dw.data_ptr(), None if dp is None else dp.data_ptr(),
                             probs.data_ptr(), experts.data_ptr(), weights.data_ptr(), out.data_ptr(), T, E, k,
                             1 if renorm else 0, 0, _st()), "router_bwd")
    return out


# ================================ communication ==================================
def allreduce_fused(st, buf, offset_elems, n, dtype, local_view, inv_scale=None, found_inf=None, prescale=1.0,
                    scale_is_reciprocal=True, ctas=None, budget_ms=None):
    """In-place fused all-reduce over symmetric buffer `buf` (see csrc/comm.cu).  A channel with device-resident
    epochs (`use_device_epochs()`) makes the launch replayable from a CUDA graph.  `budget_ms`: how long the kernel
    waits for a peer before it records an expiry and returns (default `GENESIS_COMM_TIMEOUT_MS`, 10 s)."""
    ctr = getattr(st, "epoch_dev", None)
    epoch = 0 if ctr is not None else st.next_epoch()
    budget = int(float(os.environ.get("GENESIS_COMM_TIMEOUT_MS", 10000) if budget_ms is None else budget_ms) * 1e6)
    if ctas is None:
        # enough CTAs to keep ~1.5 MB of loads in flight for big buckets, one for tiny ones
        es = torch.empty(0, dtype=dtype).element_size()
        per_rank_vecs = n * es // 16 // max(st.world, 1)
        ctas = max(1, min(int(os.environ.get("GENESIS_COMM_CTAS", 128)), (per_rank_vecs + 1023) // 1024))
    _chk(lib().gb_allreduce_fused(buf.ptr_table, st.flags.ptr_table, offset_elems, n, st.rank, st.world, epoch,
                                  float(prescale), None if inv_scale is None else inv_scale.data_ptr(),
                                  1 if scale_is_reciprocal else 0,
                                  None if found_inf is None else found_inf.data_ptr(), _DT[dtype], ctas, budget,
                                  st.status.data_ptr(), None if ctr is None else ctr.data_ptr(), _st()),
         "allreduce_fused")
    return True


def allreduce_wire(st, buf, n, dtype, out, inv_scale=None, found_inf=None, prescale=1.0, scale_is_reciprocal=True,
                   ctas=None, budget_ms=None):
    """In-place all-reduce of the float32 bucket `out` with 16-bit values on the wire: the kernel packs `out` into
    this rank's symmetric 16-bit buffer `buf` (`n` elements of `dtype`), reduces across ranks with fp32 accumulation,
    `prescale` and the overflow check, and casts the result back into `out` times 1/loss-scale (see csrc/comm.cu)."""
    ctr = getattr(st, "epoch_dev", None)
    epoch = 0 if ctr is not None else st.next_epoch()
    budget = int(float(os.environ.get("GENESIS_COMM_TIMEOUT_MS", 10000) if budget_ms is None else budget_ms) * 1e6)
    if ctas is None:
        per_rank_vecs = n * 2 // 16 // max(st.world, 1)
        ctas = max(1, min(int(os.environ.get("GENESIS_COMM_CTAS", 128)), (per_rank_vecs + 1023) // 1024))
    _chk(lib().gb_allreduce_wire(buf.ptr_table, st.flags.ptr_table, n, out.data_ptr(), st.rank, st.world, epoch,
                                 float(prescale), None if inv_scale is None else inv_scale.data_ptr(),
                                 1 if scale_is_reciprocal else 0,
                                 None if found_inf is None else found_inf.data_ptr(), _DT[dtype], ctas, budget,
                                 st.status.data_ptr(), None if ctr is None else ctr.data_ptr(), _st()),
         "allreduce_wire")


def _comm_budget():
    return int(float(os.environ.get("GENESIS_COMM_TIMEOUT_MS", 10000)) * 1e6)


def peer_pull(st, buf, send_off, send_len, recv_off, out, ctas=32):
    """All-gather / broadcast / all-to-all over peer memory (see csrc/comm.cu).  `send_off` / `send_len`:
    bytes of this rank's staged part for each destination; `recv_off`: byte offset in `out` for each source.
    `ctas` must be the same on every rank."""
    from ..distributed import symm
    W = st.world
    arr = ctypes.c_longlong * W
    _chk(lib().gb_peer_pull(buf.ptr_table, st.flags.ptr_table, arr(*send_off), arr(*send_len), arr(*recv_off),
                            out.data_ptr(), st.rank, W, st.next_epoch(), ctas, _comm_budget(),
                            st.status.data_ptr(), _st()), "peer_pull")


def peer_reduce_scatter(st, buf, out, n, scale=1.0, ctas=32):
    from ..distributed import symm
    _chk(lib().gb_peer_reduce_scatter(buf.ptr_table, st.flags.ptr_table, out.data_ptr(), n, st.rank, st.world,
                                      st.next_epoch(), float(scale), _DT[out.dtype], ctas, _comm_budget(),
                                      st.status.data_ptr(), _st()), "peer_reduce_scatter")


def peer_barrier(st):
    from ..distributed import symm
    _chk(lib().gb_peer_barrier(st.flags.ptr_table, st.rank, st.world, st.next_epoch(), _comm_budget(),
                               st.status.data_ptr(), _st()), "peer_barrier")


if torch.cuda.is_available():
    lib()


# ---- kernel families that land in their own modules ------------------------------------------
def attention_fwd(q, k, v, causal, scale):
    from . import attention
    return attention.forward(q, k, v, causal, scale)


def attention_bwd(do, q, k, v, o, lse, causal, scale):
    from . import attention
    return attention.backward(do, q, k, v, o, lse, causal, scale)


def moe_sort(experts, num_experts, align=1):
    from . import grouped
    return grouped.moe_sort(experts, num_experts, align)


def grouped_linear(x, w, offsets, out=None):
    from . import grouped
    return grouped.grouped_linear(x, w, offsets, out)


def grouped_dgrad(gy, w, offsets):
    from . import grouped
    return grouped.grouped_dgrad(gy, w, offsets)


def grouped_wgrad(gy, x, offsets, num_groups, out_dtype):
    from . import grouped
    return grouped.grouped_wgrad(gy, x, offsets, num_groups, out_dtype)


def moe_combine(y, w, pos):
    from . import grouped
    return grouped.moe_combine(y, w, pos)


def moe_combine_bwd(g, y, w, pos):
    from . import grouped
    return grouped.moe_combine_bwd(g, y, w, pos)


# =============================== sort / select / index producers ================================
_SORTABLE = (F32, F16, BF16, torch.int32)


def sort_rows(x, k, descending):
    """Stable sort along the last dim of a contiguous tensor; returns the first `k` (values, int64 indices)."""
    if x.dtype not in _SORTABLE or not x.is_contiguous() or x.dim() < 1 or x.numel() == 0:
        return NotImplemented
    cols = x.shape[-1]
    rows = x.numel() // cols
    if cols >= (1 << 30) or rows >= (1 << 31):
        return NotImplemented
    vals = torch.empty(x.shape[:-1] + (k,), dtype=x.dtype, device=x.device)
    idx = torch.empty(x.shape[:-1] + (k,), dtype=torch.int64, device=x.device)
    ws = None
    if cols > 8192:
        np2 = 1 << (cols - 1).bit_length()
        ws = torch.empty(rows * np2, dtype=torch.int64, device=x.device)
    _chk(lib().gb_sort_rows(x.data_ptr(), vals.data_ptr(), idx.data_ptr(), rows, cols, k, 1 if descending else 0,
                            _DT[x.dtype], ws.data_ptr() if ws is not None else None, _st()), "sort_rows")
    return vals, idx


def argmax_rows(x, is_min=False):
    if x.dtype not in _SORTABLE or not x.is_contiguous() or x.dim() < 1 or x.numel() == 0:
        return NotImplemented
    cols = x.shape[-1]
    out = torch.empty(x.shape[:-1], dtype=torch.int64, device=x.device)
    _chk(lib().gb_argmax_rows(x.data_ptr(), out.data_ptr(), x.numel() // cols, cols, 1 if is_min else 0,
                              _DT[x.dtype], _st()), "argmax_rows")
    return out


def bincount(idx, weights, nbins):
    if idx.dtype not in (torch.int32, torch.int64) or not idx.is_contiguous():
        return NotImplemented
    if weights is not None:
        if weights.dtype != F32 or not weights.is_contiguous():
            return NotImplemented
        out = torch.zeros(nbins, dtype=F32, device=idx.device)
    else:
        out = torch.zeros(nbins, dtype=torch.int64, device=idx.device)
    _chk(lib().gb_bincount(idx.data_ptr(), 1 if idx.dtype == torch.int64 else 0,
                           weights.data_ptr() if weights is not None else None, out.data_ptr(), idx.numel(), nbins,
                           _st()), "bincount")
    return out


def nonzero_flat(x):
    """int64 flat indices of the nonzero elements of a contiguous tensor (one host read for the count)."""
    if x.dtype not in _DT or x.dtype == torch.float64 or not x.is_contiguous():
        return NotImplemented
    n = x.numel()
    nb = (n + 1023) // 1024
    counts = torch.empty(nb + 1, dtype=torch.int32, device=x.device)
    L = lib()
    _chk(L.gb_nonzero_count(x.data_ptr(), counts.data_ptr(), n, _DT[x.dtype], _st()), "nonzero_count")
    total = int(counts[nb].item())
    out = torch.empty(total, dtype=torch.int64, device=x.device)
    if total:
        _chk(L.gb_nonzero_write(x.data_ptr(), counts.data_ptr(), out.data_ptr(), n, _DT[x.dtype], _st()), "nonzero_write")
    return out


def triu_tril(x, diag, upper):
    if not x.is_contiguous() or x.dim() < 2 or x.element_size() not in (1, 2, 4, 8) or x.numel() == 0:
        return NotImplemented
    out = torch.empty_like(x)
    _chk(lib().gb_triu_tril(x.data_ptr(), out.data_ptr(), x.numel(), x.shape[-2], x.shape[-1], int(diag),
                            1 if upper else 0, x.element_size(), _st()), "triu_tril")
    return out


def one_hot(idx, classes, dtype):
    if idx.dtype not in (torch.int32, torch.int64) or not idx.is_contiguous() or dtype not in _DT \
            or dtype in (torch.float64, torch.uint8, torch.bool):
        return NotImplemented
    out = torch.empty(idx.shape + (classes,), dtype=dtype, device=idx.device)
    _chk(lib().gb_one_hot(idx.data_ptr(), 1 if idx.dtype == torch.int64 else 0, out.data_ptr(), idx.numel(), classes,
                          _DT[dtype], _st()), "one_hot")
    return out


def arange(start, step, n, dtype, device):
    if dtype not in _DT or dtype in (torch.float64, torch.uint8, torch.bool):
        return NotImplemented
    out = torch.empty(n, dtype=dtype, device=device)
    _chk(lib().gb_arange(out.data_ptr(), n, float(start), float(step), _DT[dtype], _st()), "arange")
    return out


def repeat_interleave(x, rep, dim):
    if not x.is_contiguous() or x.element_size() not in (1, 2, 4, 8):
        return NotImplemented
    dim = dim % x.dim()
    outer = math.prod(x.shape[:dim])
    inner = math.prod(x.shape[dim + 1:])
    shape = list(x.shape)
    shape[dim] *= rep
    out = torch.empty(shape, dtype=x.dtype, device=x.device)
    _chk(lib().gb_repeat_interleave(x.data_ptr(), out.data_ptr(), outer, x.shape[dim], inner, rep, x.element_size(),
                                    _st()), "repeat_interleave")
    return out


# ================================== indexing engine ==============================
_ELEM_DT = {F32: 0, F16: 1, BF16: 2, torch.float64: 3, torch.int32: 4, torch.int64: 5, torch.uint8: 6, torch.bool: 7}
_IDX_DT = (torch.int32, torch.int64)


def _ll(vals, n):
    vals = list(vals)
    return (ctypes.c_longlong * n)(*(vals + [0] * (n - len(vals))))


def cat(tensors, dim):
    """Concatenation of contiguous tensors along `dim` in one launch per 8 inputs (tiled copies, widest element the
    alignment allows)."""
    ref = tensors[0]
    nd = ref.dim()
    if nd == 0 or any(t.dtype != ref.dtype or t.dim() != nd or not t.is_contiguous() for t in tensors):
        return NotImplemented
    dim = dim % nd
    shape = list(ref.shape)
    for t in tensors:
        if any(t.shape[d] != shape[d] for d in range(nd) if d != dim):
            return NotImplemented
    shape[dim] = sum(t.shape[dim] for t in tensors)
    out = torch.empty(shape, dtype=ref.dtype, device=ref.device)
    if out.numel() == 0:
        return out
    outer = 1
    for s_ in shape[:dim]:
        outer *= s_
    tail = 1
    for s_ in shape[dim + 1:]:
        tail *= s_
    es = ref.element_size()
    inner = [t.shape[dim] * tail for t in tensors]
    offs, pos = [], 0
    for n in inner:
        offs.append(pos)
        pos += n
    out_inner = pos
    # widen the element while every row start stays aligned
    for wide in (16, 8, 4, 2):
        if wide <= es or wide % es:
            continue
        f = wide // es
        if all(n % f == 0 for n in inner) and all(o % f == 0 for o in offs) and out_inner % f == 0 \
                and out.data_ptr() % wide == 0 and all(t.data_ptr() % wide == 0 for t in tensors):
            inner = [n // f for n in inner]
            offs = [o // f for o in offs]
            out_inner //= f
            es = wide
            break
    live = [(t, n, o) for t, n, o in zip(tensors, inner, offs) if n > 0]
    L = lib()
    for i in range(0, len(live), 8):
        chunk = live[i:i + 8]
        ptrs = (ctypes.c_void_p * len(chunk))(*[t.data_ptr() for t, _, _ in chunk])
        _chk(L.gb_cat(ptrs, _ll([n for _, n, _ in chunk], 8), _ll([o for _, _, o in chunk], 8), len(chunk),
                      out.data_ptr(), outer, out_inner, es, _st()), "cat")
    return out


def gather_dim(src, dim, index):
    nd = src.dim()
    if nd == 0 or nd > 6 or index.dim() != nd or index.dtype not in _IDX_DT or src.element_size() not in (1, 2, 4, 8):
        return NotImplemented
    dim = dim % nd
    out = torch.empty(index.shape, dtype=src.dtype, device=src.device)
    if out.numel() == 0:
        return out
    _chk(lib().gb_gather_dim(src.data_ptr(), index.data_ptr(), out.data_ptr(), nd, dim, _ll(index.shape, 6),
                             _ll(src.stride(), 6), _ll(index.stride(), 6), src.shape[dim],
                             1 if index.dtype == torch.int64 else 0, src.element_size(),
                             status_tensor(src.device).data_ptr(), _st()), "gather_dim")
    return out


def scatter_dim_(dst, dim, index, src, add):
    """dst scattered along `dim` in place from tensor or scalar `src`; `add` accumulates (atomics)."""
    nd = dst.dim()
    if nd == 0 or nd > 6 or index.dim() != nd or index.dtype not in _IDX_DT or dst.dtype not in _ELEM_DT:
        return NotImplemented
    if dst.dtype in (torch.uint8, torch.bool):
        return NotImplemented
    dim = dim % nd
    scalar = not isinstance(src, torch.Tensor)
    if not scalar and (src.dtype != dst.dtype or src.dim() != nd
                       or any(src.shape[d] < index.shape[d] for d in range(nd))):
        return NotImplemented
    if index.numel() == 0:
        return dst
    _chk(lib().gb_scatter_dim(dst.data_ptr(), index.data_ptr(), None if scalar else src.data_ptr(),
                              float(src) if scalar else 0.0, 1 if scalar else 0, 1 if add else 0, nd, dim,
                              _ll(index.shape, 6), _ll(dst.stride(), 6), _ll([0] * nd if scalar else src.stride(), 6),
                              _ll(index.stride(), 6), dst.shape[dim], 1 if index.dtype == torch.int64 else 0,
                              _ELEM_DT[dst.dtype], status_tensor(dst.device).data_ptr(), _st()), "scatter_dim")
    return dst


def _index_args(data, dims, idx, bshape, pre, post):
    """ctypes blocks of `gb_index_get / gb_index_put` (see csrc/indexing.cu): `dims` the indexed dims of `data`,
    `idx` their index tensors (broadcastable to `bshape`), `pre` / `post` the dims of `data` before / after."""
    nb = len(bshape)
    meta = (ctypes.c_int * 8)(len(idx), nb, len(pre), len(post), *[1 if t.dtype == torch.int64 else 0 for t in idx])
    d = [0] * 40
    for k, (dm, t) in enumerate(zip(dims, idx)):
        d[k] = data.shape[dm]
        d[4 + k] = data.stride(dm)
        te = t.expand(bshape)
        for b in range(nb):
            d[24 + 4 * k + b] = te.stride(b)
    for b, n in enumerate(bshape):
        d[8 + b] = n
    for j, dm in enumerate(pre):
        d[12 + j], d[15 + j] = data.shape[dm], data.stride(dm)
    for j, dm in enumerate(post):
        d[18 + j], d[21 + j] = data.shape[dm], data.stride(dm)
    ptrs = (ctypes.c_void_p * 4)(*([t.data_ptr() for t in idx] + [None] * (4 - len(idx))))
    return ptrs, meta, (ctypes.c_longlong * 40)(*d)


def index_get(data, dims, idx, bshape, pre, post):
    """out[pre, bshape, post] (contiguous) = data indexed by tensors `idx` on dims `dims`."""
    if data.element_size() not in (1, 2, 4, 8) or len(idx) > 4 or len(bshape) > 4 or len(pre) > 3 or len(post) > 3 \
            or any(t.dtype not in _IDX_DT for t in idx):
        return NotImplemented
    shape = [data.shape[d] for d in pre] + list(bshape) + [data.shape[d] for d in post]
    out = torch.empty(shape, dtype=data.dtype, device=data.device)
    if out.numel() == 0:
        return out
    ptrs, meta, dd = _index_args(data, dims, idx, bshape, pre, post)
    _chk(lib().gb_index_get(data.data_ptr(), out.data_ptr(), ptrs, meta, dd, data.element_size(),
                            status_tensor(data.device).data_ptr(), _st()), "index_get")
    return out


def index_put_(data, dims, idx, bshape, pre, post, val, add):
    """data[...] (= | +=) val, where `val` is a scalar or a contiguous tensor of shape [pre, bshape, post]."""
    if data.dtype not in _ELEM_DT or len(idx) > 4 or len(bshape) > 4 or len(pre) > 3 or len(post) > 3 \
            or any(t.dtype not in _IDX_DT for t in idx):
        return NotImplemented
    if add and data.dtype in (torch.uint8, torch.bool):
        return NotImplemented
    scalar = not isinstance(val, torch.Tensor)
    if not scalar and (val.dtype != data.dtype or not val.is_contiguous()):
        return NotImplemented
    n = 1
    for s_ in [data.shape[d] for d in pre] + list(bshape) + [data.shape[d] for d in post]:
        n *= s_
    if n == 0:
        return data
    if not scalar and val.numel() != n:
        return NotImplemented
    ptrs, meta, dd = _index_args(data, dims, idx, bshape, pre, post)
    _chk(lib().gb_index_put(data.data_ptr(), None if scalar else val.data_ptr(), float(val) if scalar else 0.0,
                            1 if scalar else 0, 1 if add else 0, ptrs, meta, dd, _ELEM_DT[data.dtype],
                            status_tensor(data.device).data_ptr(), _st()), "index_put")
    return data


def masked_fill_(a, mask, value):
    """a[mask] = value in place; `mask` (bool, contiguous) covers the leading dims of contiguous `a`."""
    if a.dtype not in _ELEM_DT or not a.is_contiguous() or mask.dtype != torch.bool or not mask.is_contiguous() \
            or tuple(a.shape[:mask.dim()]) != tuple(mask.shape):
        return NotImplemented
    rows = mask.numel()
    inner = a.numel() // rows if rows else 0
    if a.numel():
        _chk(lib().gb_masked_fill(a.data_ptr(), mask.data_ptr(), float(value), rows, inner, _ELEM_DT[a.dtype], _st()),
             "masked_fill")
    return a
