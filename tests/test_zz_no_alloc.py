"""The allocation-free RMSNorm backward (`gb_rmsnorm_bwd_noalloc`, declared in csrc/noalloc.h).

It is meant for callers that may not allocate where they run this kernel: code under a memory budget
fixed by someone else (a serving process with pre-sized pools, a plugin in a foreign runtime) and
latency-critical loops that must not hit the device-wide synchronisation of cudaMalloc / cudaFree.
The test goes through the exported C symbol with ctypes, hands it inputs and outputs only, and checks
two calls in a row (different data, different widths - the shared scratch keeps the first call's
contents) against the regular entry point.  The file name sorts last so that a failure here cannot
hide other tests from a run that stops at the first failure.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _entry():
    from genesis_b200 import _lib
    L = _lib.get(required=True)
    fn = L.gb_rmsnorm_bwd_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 6 + [ctypes.c_longlong, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    L.gb_rmsnorm_bwd_noalloc_strerror.restype = ctypes.c_char_p
    L.gb_rmsnorm_bwd_noalloc_strerror.argtypes = [ctypes.c_int]
    L.gb_rmsnorm_bwd_noalloc_max_cols.restype = ctypes.c_int
    return L, fn


def _call(fn, g, x, w, rstd):
    dx = torch.empty_like(x)
    dw = torch.empty(x.shape[-1], dtype=torch.float32, device=x.device)
    code = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}
    rc = fn(g.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dx.data_ptr(), dw.data_ptr(),
            x.numel() // x.shape[-1], x.shape[-1], code[x.dtype], code[w.dtype],
            torch.cuda.current_stream().cuda_stream)
    return rc, dx, dw


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float32])
def test_noalloc_rmsnorm_bwd_matches_regular_entry_point_twice(dt):
    from genesis_b200.ops import dispatch as K
    L, fn = _entry()
    gen = torch.Generator().manual_seed(7)
    atol = 2e-2 if dt == torch.bfloat16 else 1e-5
    for rows, cols in [(1000, 896), (333, 2048)]:          # two calls in a row on the same scratch
        x = torch.randn(rows, cols, generator=gen).to(dt).cuda()
        g = torch.randn(rows, cols, generator=gen).to(dt).cuda()
        w = (torch.randn(cols, generator=gen) * 0.1 + 1.0).cuda()
        _, rstd = K.rmsnorm_fwd(x, w, 1e-6)
        dx_ref, dw_ref = K.rmsnorm_bwd(g, x, w, rstd)       # regular entry point (caller-provided scratch)
        # (the framework's own counter: it reads whichever allocator backs torch, the native pool or torch's)
        from genesis_b200 import cuda as gcuda
        from genesis_b200.cuda import pool
        before = gcuda.memory_allocated()
        rc, dx, dw = _call(fn, g, x, w, rstd)
        assert rc == 0, L.gb_rmsnorm_bwd_noalloc_strerror(rc)
        torch.cuda.synchronize()
        # only the two outputs were allocated by the caller (each rounded up to its size class), nothing by the callee
        outs = (dx.numel() * dx.element_size(), dw.numel() * 4)
        bound = sum(pool.round_size(n) for n in outs) if pool.is_installed() else sum(outs) + 1024
        assert gcuda.memory_allocated() - before <= bound
        torch.testing.assert_close(dx.float(), dx_ref.float(), atol=atol, rtol=atol)
        torch.testing.assert_close(dw, dw_ref.float(), atol=atol * 8, rtol=atol * 4)


def test_noalloc_rejects_oversize_rows():
    L, fn = _entry()
    cols = L.gb_rmsnorm_bwd_noalloc_max_cols() + 8
    x = torch.zeros(4, cols, device="cuda", dtype=torch.bfloat16)
    w = torch.ones(cols, device="cuda")
    rstd = torch.ones(4, device="cuda")
    rc, _, _ = _call(fn, x, x, w, rstd)
    assert rc == -10
    assert b"max 4096" in L.gb_rmsnorm_bwd_noalloc_strerror(rc)
    bad = torch.zeros(4, 12, device="cuda", dtype=torch.bfloat16)
    rc, _, _ = _call(fn, bad, bad, torch.ones(12, device="cuda"), rstd)
    assert rc == -11
