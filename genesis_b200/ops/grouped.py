"""Grouped (ragged) GEMMs and the expert sort for mixture-of-experts, on the GROUP_M / GROUP_K modes of
`csrc/gemm_sm100.cu` and the counting sort of `csrc/moe.cu`.

Rows are sorted by expert into segments padded to multiples of 128 rows (one GEMM tile), so every
tile belongs to exactly one expert and the contraction of the weight-gradient GEMM never crosses a
segment boundary.  Pad rows are zero on the way in, hence zero on the way out.
"""
import torch

from . import native as N

ALIGN = 128


def _i32(t):
    return t if t.dtype == torch.int32 else t.to(torch.int32)


def moe_sort(experts, num_experts, align):
    """experts [T, k] int32 on CUDA -> (token_of [Mp] int32 with -1 in pad rows, pos [T, k] int32,
    offsets [E+1] int32), segments padded to `ALIGN` rows (`align` == 0: dense, no padding)."""
    if experts.dtype != torch.int32 or not experts.is_contiguous() or num_experts > 1024:
        return NotImplemented
    T, k = experts.shape
    pairs = T * k
    dev = experts.device
    align = 1 if align == 0 else ALIGN          # 0: dense; anything else: one GEMM tile
    max_rows = (pairs + num_experts * (align - 1) + align - 1) // align * align
    counts = _counts(experts, num_experts)
    offsets = torch.empty(num_experts + 1, dtype=torch.int32, device=dev)
    cursor = torch.empty(num_experts, dtype=torch.int32, device=dev)
    pos = torch.empty(T, k, dtype=torch.int32, device=dev)
    token_of = torch.empty(max_rows, dtype=torch.int32, device=dev)
    N._chk(N.lib().gb_moe_sort(experts.data_ptr(), counts.data_ptr(), offsets.data_ptr(), cursor.data_ptr(),
                               pos.data_ptr(), token_of.data_ptr(), pairs, k, num_experts, align, max_rows, N._st()),
           "moe_sort")
    return token_of, pos, offsets


def _counts(experts, num_experts):
    """Per-expert histogram; the router kernel already produced it for the forward pass, this is the
    stand-alone path."""
    c = getattr(experts, "_gb_counts", None)
    if c is not None:
        return c
    return torch.bincount(experts.reshape(-1).long(), minlength=num_experts).to(torch.int32)


def _ok(x, w, offsets):
    return (x.dtype in (torch.bfloat16, torch.float16) and x.dtype == w.dtype and x.is_contiguous()
            and w.is_contiguous() and w.dim() == 3 and offsets.dtype == torch.int32 and offsets.is_cuda
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and x.shape[0] % ALIGN == 0)


def _gemm(a, b, out, M, Nn, Kk, lda, ldb, strideB, strideD, a_mn, b_mn, mode, offsets, groups):
    rc = N.lib().gb_gemm(a.data_ptr(), b.data_ptr(), out.data_ptr(), None, M, Nn, Kk, 1, lda, ldb, Nn, 0, strideB,
                         strideD, a_mn, b_mn, N._GEMM_DT[a.dtype], N._GEMM_DT[out.dtype], 0, 0, 1.0, mode,
                         offsets.data_ptr(), groups, 1, 0, N.status_tensor(a.device).data_ptr(), N._sms(a.device), N._st())
    N._chk(rc, "grouped gemm")
    return out


def grouped_linear(x, w, offsets, out=None):
    """y[seg g] = x[seg g] @ w[g]^T.  x [Mp, K], w [G, N, K] -> [Mp, N] (into `out` when given)."""
    if not _ok(x, w, offsets) or x.shape[1] % 8 or w.shape[1] % 8:
        return NotImplemented
    Mp, Kk = x.shape
    G, Nn, _ = w.shape
    if out is not None and (out.dtype != x.dtype or not out.is_contiguous() or tuple(out.shape) != (Mp, Nn)
                            or out.data_ptr() % 16):
        return NotImplemented
    # every tile below offsets[-1] is written (pad rows are zero on the way in); rows past it stay unwritten
    if out is None:
        out = torch.empty(Mp, Nn, dtype=x.dtype, device=x.device)
    return _gemm(x, w, out, Mp, Nn, Kk, Kk, Kk, Nn * Kk, 0, 0, 0, 1, offsets, G)


def grouped_dgrad(gy, w, offsets):
    """dx[seg g] = gy[seg g] @ w[g].  gy [Mp, N], w [G, N, K] -> [Mp, K]."""
    if not _ok(gy, w, offsets) or gy.shape[1] % 8 or w.shape[2] % 8:
        return NotImplemented
    Mp, Nn = gy.shape
    G, _, Kk = w.shape
    out = torch.empty(Mp, Kk, dtype=gy.dtype, device=gy.device)
    # contraction over N: B operand is w[g] stored [N (contraction), K (output columns)] = MN-major
    return _gemm(gy, w, out, Mp, Kk, Nn, Nn, Kk, Nn * Kk, 0, 0, 1, 1, offsets, G)


def grouped_wgrad(gy, x, offsets, num_groups, out_dtype):
    """dw[g] = gy[seg g]^T @ x[seg g].  gy [Mp, N], x [Mp, K] -> [G, N, K] (fp32 accumulate)."""
    if gy.dtype not in (torch.bfloat16, torch.float16) or gy.dtype != x.dtype or not gy.is_contiguous() \
            or not x.is_contiguous() or offsets.dtype != torch.int32 or gy.shape[1] % 8 or x.shape[1] % 8:
        return NotImplemented
    Mp, Nn = gy.shape
    Kk = x.shape[1]
    out = torch.empty(num_groups, Nn, Kk, dtype=out_dtype or gy.dtype, device=gy.device)
    # contraction over the rows of a segment: both operands are read "transposed" (MN-major)
    return _gemm(gy, x, out, Nn, Kk, Mp, Nn, Kk, 0, Nn * Kk, 1, 1, 2, offsets, num_groups)


def moe_combine(y, w, pos):
    if y.dtype not in N._FLOATS or not y.is_contiguous() or w.dtype != torch.float32 or pos.dtype != torch.int32:
        return NotImplemented
    T, k = w.shape
    cols = y.shape[1]
    out = torch.empty(T, cols, dtype=y.dtype, device=y.device)
    rc = N.lib().gb_moe_combine(y.data_ptr(), w.contiguous().data_ptr(), pos.contiguous().data_ptr(), out.data_ptr(),
                                T, k, cols, N._DT[y.dtype], N._st())
    if rc == -2:
        return NotImplemented
    N._chk(rc, "moe_combine")
    return out


def moe_combine_bwd(g, y, w, pos):
    if y.dtype not in N._FLOATS or g.dtype != y.dtype or not g.is_contiguous() or pos.dtype != torch.int32:
        return NotImplemented
    T, k = w.shape
    cols = y.shape[1]
    dy = torch.zeros_like(y)
    dw = torch.empty(T, k, dtype=torch.float32, device=y.device)
    N._chk(N.lib().gb_moe_combine_bwd(g.data_ptr(), y.data_ptr(), w.contiguous().data_ptr(),
                                      pos.contiguous().data_ptr(), dy.data_ptr(), dw.data_ptr(), T, k, cols,
                                      N._DT[y.dtype], N._st()), "moe_combine_bwd")
    return dy, dw
