"""Flash-attention bindings (tcgen05 kernels in `csrc/attention_sm100.cu`).

q [B, S, Hq, D]; k, v [B, Sk, Hkv, D]; 16-bit dtypes; D in {64, 128}; Hkv divides Hq; Sk >= S
(a causal mask is aligned to the end of the keys).  Other inputs return NotImplemented.
"""
import ctypes

import torch

from . import native as N

_SIG_FWD = "ppppp" + "iiiiii" + "i" + "f" + "i" + "pp"
_SIG_BWD = "ppppppppppp" + "iiiiii" + "i" + "f" + "i" + "pp"
N._SIGS["gb_attn_fwd"] = _SIG_FWD
N._SIGS["gb_attn_bwd"] = _SIG_BWD
_bound = False


def _lib():
    global _bound
    L = N.lib()
    if not _bound:
        for name, sig in (("gb_attn_fwd", _SIG_FWD), ("gb_attn_bwd", _SIG_BWD)):
            fn = getattr(L, name)
            fn.argtypes = [N._C[c] for c in sig]
            fn.restype = ctypes.c_int
        _bound = True
    return L


def _supported(q, k, v):
    if q.dtype not in (torch.bfloat16, torch.float16) or k.dtype != q.dtype or v.dtype != q.dtype:
        return False
    if q.dim() != 4 or k.dim() != 4 or k.shape != v.shape:
        return False
    B, S, Hq, D = q.shape
    if D not in (64, 128) or k.shape[0] != B or k.shape[3] != D or Hq % k.shape[2] or k.shape[1] < S or S == 0:
        return False
    return all(t.is_contiguous() and t.data_ptr() % 16 == 0 for t in (q, k, v))


def forward(q, k, v, causal, scale):
    if not _supported(q, k, v):
        return NotImplemented
    B, S, Hq, D = q.shape
    Sk, Hkv = k.shape[1], k.shape[2]
    o = torch.empty_like(q)
    lse = torch.empty(B, Hq, S, dtype=torch.float32, device=q.device)
    N._chk(_lib().gb_attn_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(), B, S, Sk, Hq,
                              Hkv, D, 1 if causal else 0, float(scale), 1 if q.dtype == torch.bfloat16 else 0,
                              N.status_tensor(q.device).data_ptr(), N._st()), "attn_fwd")
    return o, lse


def backward(do, q, k, v, o, lse, causal, scale):
    if not _supported(q, k, v) or do.dtype != q.dtype or not do.is_contiguous() or not o.is_contiguous():
        return NotImplemented
    B, S, Hq, D = q.shape
    Sk, Hkv = k.shape[1], k.shape[2]
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    delta = torch.empty(B, Hq, S, dtype=torch.float32, device=q.device)
    # grouped-query attention: the query heads of a group accumulate dK / dV in fp32 scratch
    ws = torch.empty(2 * k.numel(), dtype=torch.float32, device=q.device) if Hq != Hkv else None
    N._chk(_lib().gb_attn_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), do.data_ptr(), lse.data_ptr(),
                              delta.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
                              ws.data_ptr() if ws is not None else None, B, S, Sk, Hq, Hkv, D,
                              1 if causal else 0, float(scale), 1 if q.dtype == torch.bfloat16 else 0,
                              N.status_tensor(q.device).data_ptr(), N._st()), "attn_bwd")
    return dq, dk, dv
