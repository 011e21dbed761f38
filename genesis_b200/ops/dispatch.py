"""Kernel entry points on raw `torch.Tensor`s.

One device path per device: CUDA tensors go to the sm_100a kernels of
`genesis_b200.ops.native` (hand-written CUDA loaded through ctypes); CPU tensors
use torch CPU math, which is also the numerical oracle of the test-suite (the
reference's CPU backend is the same thing, `genesis/ops/cpu/*.py`).

A native wrapper returns `NotImplemented` for a layout/dtype it does not cover
(e.g. float64 or >4-D strided broadcasting); only then is the generic torch op
used on CUDA.
"""
import collections
import math
import os

import torch

from . import native as N

_F32 = torch.float32
_LOW = (torch.float16, torch.bfloat16)

# ---- falling off the native path is counted, and an error in strict mode ---------------------------------------
# Every op below tries its sm_100a kernel first; when the wrapper answers `NotImplemented` (a dtype / layout the
# kernel family does not cover) a CUDA tensor is handed to the generic torch op instead.  That is legitimate for
# rare cases (float64, integer arithmetic) and invisible in a benchmark, so it is counted per op here;
# `GENESIS_STRICT_NATIVE=1` (or `strict_native(True)`) turns such a fall into an error.  bench.py and the GPU model
# tests assert that the counter stays at zero on the paths they time.
fallbacks = collections.Counter()
_strict = [os.environ.get("GENESIS_STRICT_NATIVE", "0") == "1"]


def _fell(op):
    fallbacks[op] += 1
    if _strict[0]:
        raise RuntimeError(f"GENESIS_STRICT_NATIVE: op '{op}' has no native sm_100a path for these arguments and "
                           f"would have run a library kernel")


def _fb(t, op):
    """Marks a fall to the library op when `t` is a non-empty CUDA tensor (for ops whose native branch is guarded by
    more than the device test)."""
    if isinstance(t, torch.Tensor) and t.is_cuda and t.numel() > 0:
        _fell(op)


def fallback_counts():
    """{op name: times a CUDA call was served by a library kernel instead of a native one} since the last reset."""
    return dict(fallbacks)


def reset_fallbacks():
    fallbacks.clear()


class strict_native:
    """`with strict_native():` raises on any CUDA op that would leave the native path (also usable as a switch:
    `strict_native.set(True)`)."""

    def __init__(self, on=True):
        self.on, self.prev = on, None

    def __enter__(self):
        self.prev, _strict[0] = _strict[0], self.on
        return self

    def __exit__(self, *exc):
        _strict[0] = self.prev
        return False

    @staticmethod
    def set(on):
        _strict[0] = bool(on)


def _cuda(t):
    return t.is_cuda


# =============================== data movement ===================================
def to_dtype(t, dtype):
    if t.dtype == dtype:
        return t
    if t.is_cuda:
        r = N.cast(t, dtype)
        if r is not NotImplemented:
            return r
        _fell("to_dtype")
    return t.to(dtype)


def copy_(dst, src):
    if dst.is_cuda and src.is_cuda:
        r = N.copy_(dst, src)
        if r is not NotImplemented:
            return dst
        _fell("copy_")
    dst.copy_(src)
    return dst


def contiguous(t):
    if t.is_contiguous():
        return t
    if t.is_cuda:
        r = N.contiguous(t)
        if r is not NotImplemented:
            return r
        _fell("contiguous")
    return t.contiguous()


def clone(t):
    if t.is_cuda:
        out = torch.empty(t.shape, dtype=t.dtype, device=t.device)
        copy_(out, t)
        return out
    return t.clone(memory_format=torch.contiguous_format)


def fill_(t, value):
    if t.is_cuda:
        r = N.fill_(t, value)
        if r is not NotImplemented:
            return t
        _fell("fill_")
    t.fill_(value)
    return t


def transpose_into(dst, src):
    """dst [C, R] <- src [R, C] transposed (both contiguous)."""
    if src.is_cuda:
        r = N.transpose_into(dst, src)
        if r is not NotImplemented:
            return dst
        _fell("transpose_into")
    dst.copy_(src.t())
    return dst


def zero_(t):
    return fill_(t, 0)


def fill_view_(v, value):
    """`v[...] = value` for a strided view: contiguous float views take the fill kernel, the rest the strided-copy
    kernel fed from a one-element tensor broadcast through zero strides."""
    if not v.is_cuda:
        v.fill_(value)
        return v
    if N.fill_(v, value) is not NotImplemented:
        return v
    if v.dim() == 0 or v.dim() > 6 or v.element_size() not in (1, 2, 4, 8) or v.is_complex():
        return NotImplemented
    one = torch.tensor([value], dtype=v.dtype).to(v.device, non_blocking=False)
    return v if N.copy_(v, one.expand(v.shape)) is not NotImplemented else NotImplemented


# ================================ elementwise ====================================
def _binary(name, torch_fn, a, b):
    ta = a if isinstance(a, torch.Tensor) else b
    if ta.is_cuda:
        r = N.binary(name, a, b)
        if r is not NotImplemented:
            return r
        _fell(name)
    return torch_fn(a, b)


def add(a, b):
    return _binary("add", torch.add, a, b)


def sub(a, b):
    return _binary("sub", torch.sub, a, b)


def mul(a, b):
    return _binary("mul", torch.mul, a, b)


def div(a, b):
    return _binary("div", torch.true_divide, a, b)


def maximum(a, b):
    return _binary("max", torch.maximum, a, b)


def minimum(a, b):
    return _binary("min", torch.minimum, a, b)


def add_(a, b):
    """a += b (same shape)."""
    if a.is_cuda and isinstance(b, torch.Tensor):
        r = N.add_(a, b)
        if r is not NotImplemented:
            return a
        _fell("add_")
    a.add_(b)
    return a


def axpy_(a, b, alpha):
    """a += alpha * b."""
    if a.is_cuda:
        r = N.add_(a, b, alpha)
        if r is not NotImplemented:
            return a
        _fell("axpy_")
    a.add_(b, alpha=alpha)
    return a


def mul_(a, b):
    if a.is_cuda:
        r = N.mul_(a, b)
        if r is not NotImplemented:
            return a
        _fell("mul_")
    a.mul_(b)
    return a


_UNARY_TORCH = {
    "neg": torch.neg, "exp": torch.exp, "log": torch.log, "sqrt": torch.sqrt, "rsqrt": torch.rsqrt,
    "sin": torch.sin, "cos": torch.cos, "tanh": torch.tanh, "sigmoid": torch.sigmoid,
    "relu": torch.relu, "abs": torch.abs, "sign": torch.sign,
    "silu": torch.nn.functional.silu,
    "gelu": lambda x: torch.nn.functional.gelu(x, approximate="tanh"),
    "reciprocal": torch.reciprocal,
}


def unary(name, t):
    if t.is_cuda:
        r = N.unary(name, t)
        if r is not NotImplemented:
            return r
        _fell(name)
    return _UNARY_TORCH[name](t)


def unary_bwd(name, g, x, y=None):
    """dL/dx for y = f(x), given g = dL/dy. `y` is passed where cheaper (exp, sqrt, tanh, sigmoid)."""
    if g.is_cuda:
        r = N.unary_bwd(name, g, x if x is not None else y, y)
        if r is not NotImplemented:
            return r
        _fell(name + "_bwd")
    if name == "neg":
        return -g
    if name == "exp":
        return g * y
    if name == "log":
        return g / x
    if name == "sqrt":
        return g / (2 * y)
    if name == "sin":
        return g * torch.cos(x)
    if name == "cos":
        return -g * torch.sin(x)
    if name == "tanh":
        return g * (1 - y * y)
    if name == "sigmoid":
        return g * y * (1 - y)
    if name == "relu":
        return g * (x > 0).to(g.dtype)
    if name == "abs":
        return g * torch.sign(x)
    if name == "silu":
        xf = x.float()
        s = torch.sigmoid(xf)
        return (g.float() * (s * (1 + xf * (1 - s)))).to(g.dtype)
    if name == "gelu":
        xf = x.float()
        c = math.sqrt(2.0 / math.pi)
        inner = c * (xf + 0.044715 * xf ** 3)
        th = torch.tanh(inner)
        d = 0.5 * (1 + th) + 0.5 * xf * (1 - th * th) * c * (1 + 3 * 0.044715 * xf * xf)
        return (g.float() * d).to(g.dtype)
    raise KeyError(name)


def pow_scalar(t, p):
    if t.is_cuda:
        r = N.scalar_op("pow", t, p)
        if r is not NotImplemented:
            return r
        _fell("pow_scalar")
    return torch.pow(t, p)


def rpow_scalar(t, base):
    if t.is_cuda:
        r = N.scalar_op("rpow", t, base)
        if r is not NotImplemented:
            return r
        _fell("rpow_scalar")
    return torch.pow(torch.tensor(base, dtype=t.dtype, device=t.device), t)


def clamp(t, lo, hi):
    if t.is_cuda:
        r = N.clamp(t, lo, hi)
        if r is not NotImplemented:
            return r
        _fell("clamp")
    return torch.clamp(t, lo, hi)


def where(c, a, b):
    if c.is_cuda:
        r = N.where(c, a, b)
        if r is not NotImplemented:
            return r
        _fell("where")
    if not isinstance(a, torch.Tensor):
        ref = b if isinstance(b, torch.Tensor) else None
        a = torch.tensor(a, dtype=ref.dtype if ref is not None else torch.float32, device=c.device)
    if not isinstance(b, torch.Tensor):
        b = torch.tensor(b, dtype=a.dtype, device=c.device)
    return torch.where(c, a, b)


_CMP_TORCH = {"eq": torch.eq, "ne": torch.ne, "lt": torch.lt, "le": torch.le, "gt": torch.gt, "ge": torch.ge}


def compare(name, a, b):
    if a.is_cuda:
        r = N.compare(name, a, b)
        if r is not NotImplemented:
            return r
        _fell(name)
    return _CMP_TORCH[name](a, b)


# ================================= reductions ====================================
def _norm_dims(t, dims):
    if dims is None:
        return None
    if isinstance(dims, int):
        dims = (dims,)
    return tuple(sorted(d % max(t.dim(), 1) for d in dims))


def reduce(name, t, dims=None, keepdim=False):
    """sum / mean / max / min over `dims` (None = all). max/min return values only."""
    dims = _norm_dims(t, dims)
    if t.is_cuda:
        r = N.reduce(name, t, dims, keepdim)
        if r is not NotImplemented:
            return r
        _fell("reduce_" + name)
    if name in ("sum", "mean"):
        fn = torch.sum if name == "sum" else torch.mean
        if dims is None:
            out = fn(t)
            return out.reshape((1,) * t.dim()) if keepdim else out
        return fn(t, dim=dims, keepdim=keepdim)
    fn = torch.amax if name == "max" else torch.amin
    if dims is None:
        out = fn(t)
        return out.reshape((1,) * t.dim()) if keepdim else out
    return fn(t, dim=dims, keepdim=keepdim)


def sum_to_shape(t, shape):
    """Sum broadcast dimensions of `t` so that the result has `shape`."""
    shape = tuple(shape)
    if tuple(t.shape) == shape:
        return t
    lead = t.dim() - len(shape)
    dims = list(range(lead))
    for i, s in enumerate(shape):
        if s == 1 and t.shape[lead + i] != 1:
            dims.append(lead + i)
    out = reduce("sum", t, tuple(dims), keepdim=True) if dims else t
    return out.reshape(shape)


# ================================== matmul =======================================
def matmul(a, b):
    if a.is_cuda:
        r = N.matmul(a, b)
        if r is not NotImplemented:
            return r
        _fell("matmul")
    return torch.matmul(a, b)


def linear(x, w, bias=None, out_dtype=None):
    """y = x @ w.T (+ bias); x [..., K], w [N, K]."""
    if x.is_cuda:
        r = N.linear(x, w, bias, out_dtype)
        if r is not NotImplemented:
            return r
        _fell("linear")
    y = torch.nn.functional.linear(x, w, None if bias is None else bias.to(x.dtype))
    return y if out_dtype is None else y.to(out_dtype)


def linear_dgrad(gy, w):
    """dx = gy @ w; gy [..., N], w [N, K].  When the optimizer keeps a [K, N] twin of `w` current
    (`amp_state.transposed_of`), the GEMM reads that instead: K-major operands on both sides."""
    from ..amp_state import transposed_of
    wt = transposed_of(w)
    if wt is not None and gy.dtype == wt.dtype:
        return linear(gy, wt)
    if gy.is_cuda:
        r = N.linear_dgrad(gy, w)
        if r is not NotImplemented:
            return r
        _fell("linear_dgrad")
    return torch.matmul(gy, w)


def linear_wgrad(gy, x, out_dtype=None, accum=None, out=None):
    """dw = gy^T @ x over all leading dims; optional `accum` ([N, K]) gets += dw in place, optional `out` ([N, K])
    receives dw (a gradient slot that already exists, e.g. a DDP bucket view)."""
    if gy.is_cuda:
        r = N.linear_wgrad(gy, x, out_dtype, accum, out)
        if r is not NotImplemented:
            return r
        _fell("linear_wgrad")
    g2 = gy.reshape(-1, gy.shape[-1])
    x2 = x.reshape(-1, x.shape[-1])
    dw = torch.matmul(g2.t().float(), x2.float()) if g2.dtype in _LOW else torch.matmul(g2.t(), x2)
    if accum is not None:
        accum.add_(dw.to(accum.dtype))
        return accum
    if out is not None:
        out.copy_(dw.reshape(out.shape))
        return out
    return dw.to(out_dtype or gy.dtype)


def bias_grad(gy, out_dtype=None):
    """db = sum of gy over all leading dims (fp32 accumulate)."""
    g2 = gy.reshape(-1, gy.shape[-1])
    r = reduce("sum", g2.float() if (not g2.is_cuda and g2.dtype in _LOW) else g2, (0,), False)
    return r.to(out_dtype or gy.dtype)


# ============================= normalisation / softmax ===========================
def rmsnorm_fwd(x, w, eps):
    """Returns (y, rstd[rows] fp32)."""
    if x.is_cuda:
        r = N.rmsnorm_fwd(x, w, eps)
        if r is not NotImplemented:
            return r
        _fell("rmsnorm_fwd")
    xf = x.float()
    rstd = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    y = (xf * rstd * w.float()).to(x.dtype)
    return y, rstd.reshape(-1)


def rmsnorm_bwd(g, x, w, rstd):
    """Returns (dx, dw fp32)."""
    if g.is_cuda:
        r = N.rmsnorm_bwd(g, x, w, rstd)
        if r is not NotImplemented:
            return r
        _fell("rmsnorm_bwd")
    n = x.shape[-1]
    xf, gf, wf = x.float(), g.float(), w.float()
    rs = rstd.reshape(*x.shape[:-1], 1)
    xhat = xf * rs
    gw = gf * wf
    dx = rs * (gw - xhat * (gw * xhat).sum(-1, keepdim=True) / n)
    dw = (gf * xhat).reshape(-1, n).sum(0)
    return dx.to(x.dtype), dw


def add_rmsnorm_fwd(x, res, w, eps):
    """Returns (s = x + res in x's dtype, rmsnorm(s) * w, rstd[rows] fp32): residual addition and the normalisation
    that follows it in one pass."""
    if x.is_cuda:
        r = N.add_rmsnorm_fwd(x, res, w, eps)
        if r is not NotImplemented:
            return r
        _fell("add_rmsnorm_fwd")
    s = add(x, res)
    y, rstd = rmsnorm_fwd(s, w, eps)
    return s, y, rstd


def add_rmsnorm_bwd(g, gres, x, w, rstd):
    """Returns (rmsnorm_backward(g) + gres, dw fp32)."""
    if g.is_cuda:
        r = N.add_rmsnorm_bwd(g, gres, x, w, rstd)
        if r is not NotImplemented:
            return r
        _fell("add_rmsnorm_bwd")
    dx, dw = rmsnorm_bwd(g, x, w, rstd)
    return add(dx, gres), dw


def layernorm_fwd(x, w, b, eps):
    """Returns (y, mean[rows], rstd[rows])."""
    if x.is_cuda:
        r = N.layernorm_fwd(x, w, b, eps)
        if r is not NotImplemented:
            return r
        _fell("layernorm_fwd")
    xf = x.float()
    mean = xf.mean(-1, keepdim=True)
    var = xf.var(-1, unbiased=False, keepdim=True)
    rstd = torch.rsqrt(var + eps)
    y = (xf - mean) * rstd
    if w is not None:
        y = y * w.float()
    if b is not None:
        y = y + b.float()
    return y.to(x.dtype), mean.reshape(-1), rstd.reshape(-1)


def layernorm_bwd(g, x, w, mean, rstd):
    """Returns (dx, dw fp32, db fp32)."""
    if g.is_cuda:
        r = N.layernorm_bwd(g, x, w, mean, rstd)
        if r is not NotImplemented:
            return r
        _fell("layernorm_bwd")
    n = x.shape[-1]
    xf, gf = x.float(), g.float()
    mu = mean.reshape(*x.shape[:-1], 1)
    rs = rstd.reshape(*x.shape[:-1], 1)
    xhat = (xf - mu) * rs
    gw = gf * w.float() if w is not None else gf
    dx = rs * (gw - gw.mean(-1, keepdim=True) - xhat * (gw * xhat).mean(-1, keepdim=True))
    dw = (gf * xhat).reshape(-1, n).sum(0)
    db = gf.reshape(-1, n).sum(0)
    return dx.to(x.dtype), dw, db


def softmax_fwd(x, dim, log=False):
    if x.is_cuda:
        r = N.softmax_fwd(x, dim, log)
        if r is not NotImplemented:
            return r
        _fell("softmax_fwd")
    return torch.log_softmax(x, dim) if log else torch.softmax(x, dim)


def softmax_bwd(g, y, dim, log=False):
    if g.is_cuda:
        r = N.softmax_bwd(g, y, dim, log)
        if r is not NotImplemented:
            return r
        _fell("softmax_bwd")
    if log:
        return g - torch.exp(y) * g.sum(dim, keepdim=True)
    return y * (g - (g * y).sum(dim, keepdim=True))


def cross_entropy_fwd(logits, target, ignore_index):
    """Per-row loss (fp32, 0 where ignored) and log-sum-exp (fp32). logits [N, C]."""
    if logits.is_cuda:
        r = N.cross_entropy_fwd(logits, target, ignore_index)
        if r is not NotImplemented:
            return r
        _fell("cross_entropy_fwd")
    lf = logits.float()
    lse = torch.logsumexp(lf, -1)
    valid = target != ignore_index
    tgt = torch.where(valid, target, torch.zeros_like(target))
    picked = lf.gather(1, tgt.reshape(-1, 1).long()).reshape(-1)
    loss = torch.where(valid, lse - picked, torch.zeros_like(lse))
    return loss, lse


def cross_entropy_bwd(logits, target, lse, grad_rows, ignore_index, inplace=False):
    """dlogits = (softmax - onehot) * grad_rows[row]; zero for ignored rows."""
    if logits.is_cuda:
        r = N.cross_entropy_bwd(logits, target, lse, grad_rows, ignore_index, inplace)
        if r is not NotImplemented:
            return r
        _fell("cross_entropy_bwd")
    lf = logits.float()
    p = torch.exp(lf - lse.reshape(-1, 1))
    valid = target != ignore_index
    tgt = torch.where(valid, target, torch.zeros_like(target)).long()
    p.scatter_add_(1, tgt.reshape(-1, 1), -torch.ones_like(lse).reshape(-1, 1))
    p = p * (grad_rows * valid.to(grad_rows.dtype)).reshape(-1, 1)
    return p.to(logits.dtype)


# ============================== transformer pieces ===============================
def swiglu_fwd(gate, up):
    if gate.is_cuda:
        r = N.swiglu_fwd(gate, up)
        if r is not NotImplemented:
            return r
        _fell("swiglu_fwd")
    return (torch.nn.functional.silu(gate.float()) * up.float()).to(gate.dtype)


def swiglu_bwd(g, gate, up):
    if g.is_cuda:
        r = N.swiglu_bwd(g, gate, up)
        if r is not NotImplemented:
            return r
        _fell("swiglu_bwd")
    gf, a, b = g.float(), gate.float(), up.float()
    s = torch.sigmoid(a)
    dgate = gf * b * s * (1 + a * (1 - s))
    dup = gf * a * s
    return dgate.to(gate.dtype), dup.to(up.dtype)


def swiglu_fused_fwd(gu):
    """gu [..., 2 I] holding gate | up (the output of a fused gate/up projection) -> silu(gate) * up."""
    if gu.is_cuda:
        r = N.swiglu_fused_fwd(gu)
        if r is not NotImplemented:
            return r
        _fell("swiglu_fused_fwd")
    I = gu.shape[-1] // 2
    g, u = gu[..., :I].float(), gu[..., I:].float()
    return (torch.nn.functional.silu(g) * u).to(gu.dtype)


def linear_swiglu(x, w):
    """(gu, h) with gu = x @ w^T (w the stacked [2 I, K] gate | up weight) and h = silu(gate) * up: on CUDA one GEMM
    on CTA pairs whose epilogue applies the activation; elsewhere the GEMM followed by the SwiGLU kernel."""
    if x.is_cuda:
        r = N.linear_swiglu(x, w)
        if r is not NotImplemented:
            return r
    gu = linear(x, w)
    return gu, swiglu_fused_fwd(gu if gu.is_contiguous() else contiguous(gu))


def dgrad_swiglu_bwd(gy, wd, gu):
    """d(gate | up) from the output gradient `gy` of the down projection (weight `wd` [H, I]) and gate | up `gu`:
    dh = gy @ wd, then the SwiGLU backward.  With a K-major twin of `wd` at hand (kept by the optimizer) both run as
    one GEMM whose epilogue applies the activation gradient; otherwise as a GEMM and an elementwise pass."""
    if gy.is_cuda:
        from ..amp_state import transposed_of
        wt = transposed_of(wd)
        if wt is not None:
            r = N.dgrad_swiglu_bwd(gy, wt, gu)
            if r is not NotImplemented:
                return r
    dh = linear_dgrad(gy, wd)
    return swiglu_fused_bwd(dh if dh.is_contiguous() else contiguous(dh), gu)


def swiglu_fused_bwd(dy, gu):
    """-> d(gate | up) [..., 2 I]."""
    if gu.is_cuda:
        r = N.swiglu_fused_bwd(dy, gu)
        if r is not NotImplemented:
            return r
        _fell("swiglu_fused_bwd")
    I = gu.shape[-1] // 2
    g, u, d = gu[..., :I].float(), gu[..., I:].float(), dy.float()
    sg = torch.sigmoid(g)
    return torch.cat((d * u * sg * (1 + g * (1 - sg)), d * g * sg), -1).to(gu.dtype)


def qkv_rope_split(y, cos, sin, positions, Hq, Hkv, D):
    """(rope(q), rope(k), v) from a fused projection's output y [B, S, (Hq + 2 Hkv) D] in one kernel, or None when the
    fused kernel does not apply (the caller then rotates the head groups one by one)."""
    if y.is_cuda:
        r = N.qkv_rope(y, None, None, None, cos, sin, positions, Hq, Hkv, D, False)
        if r is not NotImplemented:
            return r[1], r[2], r[3]
    return None


def qkv_rope_merge(gq, gk, gv, cos, sin, positions, Hq, Hkv, D):
    """Gradient of `qkv_rope_split`: [B, S, (Hq + 2 Hkv) D] from the three gradients in one kernel, or None."""
    if gq is not None and gq.is_cuda:
        r = N.qkv_rope(None, gq, gk, gv, cos, sin, positions, Hq, Hkv, D, True)
        if r is not NotImplemented:
            return r[0]
    return None


def rope_fwd(x, cos, sin, positions=None, inverse=False, out=None):
    """Rotate-half RoPE on x [B, S, H, D]; cos/sin [max_pos, D] (halves duplicated).
    `inverse=True` applies the transposed rotation (the backward).  `x` may be a column slice of a wider matrix
    (a fused projection's output) and `out` a slice to write into."""
    if x.is_cuda:
        r = N.rope(x, cos, sin, positions, inverse, out)
        if r is not NotImplemented:
            return r
        _fell("rope_fwd")
    B, S, H, D = x.shape
    if positions is None:
        c, s = cos[:S].reshape(1, S, 1, D), sin[:S].reshape(1, S, 1, D)
    else:
        c, s = cos[positions].reshape(B, S, 1, D), sin[positions].reshape(B, S, 1, D)
    xf = x.float()
    c, s = c.float(), s.float()
    if inverse:
        s = -s
    x1, x2 = xf[..., : D // 2], xf[..., D // 2:]
    rot = torch.cat((-x2, x1), -1)
    res = (xf * c + rot * s).to(x.dtype)
    if out is not None:
        out.copy_(res)
        return out
    return res


def embedding_fwd(weight, idx):
    if weight.is_cuda:
        r = N.embedding_fwd(weight, idx)
        if r is not NotImplemented:
            return r
        _fell("embedding_fwd")
    return weight[idx.long()]


def embedding_bwd(g, idx, num_rows, out_dtype=None):
    """Accumulating scatter of g rows into a [num_rows, D] gradient (duplicates add up)."""
    if g.is_cuda:
        r = N.embedding_bwd(g, idx, num_rows, out_dtype)
        if r is not NotImplemented:
            return r
        _fell("embedding_bwd")
    D = g.shape[-1]
    out = torch.zeros(num_rows, D, dtype=torch.float32, device=g.device)
    out.index_add_(0, idx.reshape(-1).long(), g.reshape(-1, D).float())
    return out.to(out_dtype or g.dtype)


def embedding_bwd_into(acc, g, idx):
    """acc[idx[i]] += g[i] in place: the embedding gradient added to an existing dense gradient (tied weights)
    without materialising a second [num_rows, D] tensor."""
    D = g.shape[-1]
    g2 = g.reshape(-1, D)
    g2 = g2 if g2.is_contiguous() else g2.contiguous()
    flat = idx.reshape(-1)
    flat = flat if flat.is_contiguous() else flat.contiguous()
    if g.is_cuda:
        r = N.scatter_add_rows_into(g2, flat, acc)
        if r is not NotImplemented:
            return
        _fell("embedding_bwd_into")
    acc.index_add_(0, flat.long(), g2.to(acc.dtype))


def attention_fwd(q, k, v, causal, scale):
    """q [B, S, Hq, D], k/v [B, S, Hkv, D] -> (o [B, S, Hq, D], lse [B, Hq, S] fp32, natural log)."""
    if q.is_cuda:
        r = N.attention_fwd(q, k, v, causal, scale)
        if r is not NotImplemented:
            return r
        _fell("attention_fwd")
    B, S, Hq, D = q.shape
    Sk, Hkv = k.shape[1], k.shape[2]
    g = Hq // Hkv
    qf = q.float().permute(0, 2, 1, 3)
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(g, 1)
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(g, 1)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    if causal:
        mask = torch.ones(S, Sk, dtype=torch.bool, device=q.device).tril(Sk - S)
        s = s.masked_fill(~mask, float("-inf"))
    lse = torch.logsumexp(s, -1)
    p = torch.exp(s - lse.unsqueeze(-1))
    o = torch.matmul(p, vf).permute(0, 2, 1, 3).contiguous()
    return o.to(q.dtype), lse


def attention_bwd(do, q, k, v, o, lse, causal, scale):
    if q.is_cuda:
        r = N.attention_bwd(do, q, k, v, o, lse, causal, scale)
        if r is not NotImplemented:
            return r
        _fell("attention_bwd")
    B, S, Hq, D = q.shape
    Sk, Hkv = k.shape[1], k.shape[2]
    g = Hq // Hkv
    qf = q.float().permute(0, 2, 1, 3)
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(g, 1)
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(g, 1)
    dof = do.float().permute(0, 2, 1, 3)
    of = o.float().permute(0, 2, 1, 3)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    if causal:
        mask = torch.ones(S, Sk, dtype=torch.bool, device=q.device).tril(Sk - S)
        s = s.masked_fill(~mask, float("-inf"))
    p = torch.exp(s - lse.unsqueeze(-1))
    dv = torch.matmul(p.transpose(-1, -2), dof)
    dp = torch.matmul(dof, vf.transpose(-1, -2))
    delta = (dof * of).sum(-1, keepdim=True)
    ds = p * (dp - delta) * scale
    dq = torch.matmul(ds, kf)
    dk = torch.matmul(ds.transpose(-1, -2), qf)
    dk = dk.reshape(B, Hkv, g, Sk, D).sum(2)
    dv = dv.reshape(B, Hkv, g, Sk, D).sum(2)
    return (dq.permute(0, 2, 1, 3).contiguous().to(q.dtype),
            dk.permute(0, 2, 1, 3).contiguous().to(k.dtype),
            dv.permute(0, 2, 1, 3).contiguous().to(v.dtype))


# ================================== random =======================================
def dropout_mask_apply(x, p, seed, offset):
    """y = x * keep / (1-p), keep ~ Bernoulli(1-p) from Philox(seed, offset). Returns (y, mask uint8)."""
    if x.is_cuda:
        r = N.dropout_fwd(x, p, seed, offset)
        if r is not NotImplemented:
            return r
        _fell("dropout_mask_apply")
    # Same draw and arithmetic order as the reference's CPU dropout (`nn/modules/dropout.py:16-22`):
    # u ~ U[0,1), keep where u <= 1-p, y = x * keep / (1-p).
    keep = (torch.rand(x.shape, device=x.device) <= (1.0 - p))
    return (x * keep.to(x.dtype)) / (1.0 - p), keep.to(torch.uint8)


def random_fill(kind, shape, dtype, device, seed, offset, a=0.0, b=1.0):
    """kind: 'uniform' in [a, b), 'normal' mean a std b, 'randint' integers in [a, b)."""
    dev = torch.device(device)
    if dev.type == "cuda":
        r = N.random_fill(kind, shape, dtype, dev, seed, offset, a, b)
        if r is not NotImplemented:
            return r
        _fell("random_fill")
    if kind == "uniform":
        return torch.rand(shape, dtype=torch.float32, device=dev).mul_(b - a).add_(a).to(dtype)
    if kind == "normal":
        return torch.randn(shape, dtype=torch.float32, device=dev).mul_(b).add_(a).to(dtype)
    return torch.randint(int(a), int(b), shape, device=dev).to(dtype)


# ================================== optimisers ===================================
def adamw_step(params, grads, ms, vs, lr, beta1, beta2, eps, weight_decay, step, decoupled=True,
               grad_scale=None, found_inf=None, shadows=None, dyn=None, advance=True):
    """Multi-tensor Adam/AdamW over lists of tensors, in place.

    decoupled=True: p *= 1 - lr*wd, then Adam update (AdamW, reference `optim/adamw.py:9-64`);
    decoupled=False: g += wd * p (Adam with L2, reference `optim/optimizer.py:95-150`).
    `grad_scale` (1-elem fp32 tensor) multiplies gradients; `found_inf` (1-elem fp32
    tensor, non-zero = skip) turns the whole step into a no-op without a host sync.
    `shadows`: optional low-precision copies of the parameters refreshed by the same pass.
    `advance=False`: a further launch of the SAME step (its parameters are updated with the step count and bias
    corrections the first launch advanced `dyn` to).
    """
    if params and params[0].is_cuda:
        r = N.adamw_step(params, grads, ms, vs, lr, beta1, beta2, eps, weight_decay, step, decoupled,
                         grad_scale, found_inf, shadows, dyn, advance)
        if r is not NotImplemented:
            return
        _fell("adamw_step")
    if dyn is not None:
        raise RuntimeError("capturable optimizer state needs contiguous fp32 CUDA parameters and floating-point gradients")
    if found_inf is not None and float(found_inf.item()) != 0.0:
        return
    bc1 = 1.0 - beta1 ** step
    bc2 = 1.0 - beta2 ** step
    for i, (p, g, m, v) in enumerate(zip(params, grads, ms, vs)):
        g = g.to(torch.float32) if g.dtype != p.dtype else g
        if grad_scale is not None:
            g = g * grad_scale.to(g.dtype)
        if decoupled:
            if weight_decay != 0:
                p.mul_(1.0 - lr * weight_decay)
        elif weight_decay != 0:
            g = g + weight_decay * p
        m.mul_(beta1).add_(g, alpha=1.0 - beta1)
        v.mul_(beta2).addcmul_(g, g, value=1.0 - beta2)
        mhat = m / bc1
        vhat = v / bc2
        p.sub_(lr * mhat / (vhat.sqrt() + eps))
        if shadows is not None and shadows[i] is not None:
            shadows[i].copy_(p)


def sgd_step(params, grads, bufs, lr, momentum, weight_decay):
    """u = momentum*u + (1-momentum)*(g + wd*p); p -= lr*u (reference `optim/optimizer.py:56-92`)."""
    if params and params[0].is_cuda:
        r = N.sgd_step(params, grads, bufs, lr, momentum, weight_decay)
        if r is not NotImplemented:
            return
        _fell("sgd_step")
    for p, g, u in zip(params, grads, bufs):
        g = g.to(p.dtype)
        if weight_decay != 0:
            g = g + weight_decay * p
        u.mul_(momentum).add_(g, alpha=1.0 - momentum)
        p.sub_(lr * u)


def unscale_and_check(grads, inv_scale, found_inf):
    """grads *= inv_scale in place (skipped when None); found_inf (1-elem fp32) set to 1 if any value is non-finite."""
    if grads and grads[0].is_cuda:
        r = N.unscale_and_check(grads, inv_scale, found_inf)
        if r is not NotImplemented:
            return
        _fell("unscale_and_check")
    bad = False
    for g in grads:
        if inv_scale is not None:
            g.mul_(inv_scale.to(g.dtype) if isinstance(inv_scale, torch.Tensor) else inv_scale)
        if not bool(torch.isfinite(g).all()):
            bad = True
    if bad:
        found_inf.fill_(1.0)


def scale_grads_(grads, scale):
    """Every gradient *= scale (a float or a 1-elem fp32 device tensor), one multi-tensor launch on CUDA."""
    if grads and grads[0].is_cuda:
        r = N._grad_multi(grads, scale, None, None, 1)
        if r is not NotImplemented:
            return
        _fell("scale_grads_")
    for g in grads:
        g.mul_(scale.to(g.dtype) if isinstance(scale, torch.Tensor) else scale)


def grad_norm_sq(grads, out):
    """out (1-elem fp32) += sum of squares of all grads."""
    if grads and grads[0].is_cuda:
        r = N.grad_norm_sq(grads, out)
        if r is not NotImplemented:
            return
        _fell("grad_norm_sq")
    tot = sum(float(g.float().pow(2).sum()) for g in grads)
    out.add_(tot)


# =================================== MoE =========================================
def moe_router(logits, k, renorm):
    """softmax over experts, top-k, optional renormalisation.
    Returns (weights [T,k] fp32, experts [T,k] int32, probs [T,E] fp32, counts [E] int32)."""
    if logits.is_cuda:
        r = N.moe_router(logits, k, renorm)
        if r is not NotImplemented:
            return r
        _fell("moe_router")
    probs = torch.softmax(logits.float(), -1)
    w, e = torch.topk(probs, k, dim=-1, sorted=False)
    if renorm:
        w = w / (w.sum(-1, keepdim=True) + 1e-20)
    counts = torch.bincount(e.reshape(-1), minlength=logits.shape[-1]).to(torch.int32)
    return w, e.to(torch.int32), probs, counts


def moe_router_bwd(dweights, dprobs, probs, experts, weights, renorm):
    """Gradient of `moe_router` w.r.t. the logits. `dweights` [T,k] / `dprobs` [T,E] may be None."""
    if probs.is_cuda:
        r = N.moe_router_bwd(dweights, dprobs, probs, experts, weights, renorm)
        if r is not NotImplemented:
            return r
        _fell("moe_router_bwd")
    idx = experts.long()
    total = torch.zeros_like(probs) if dprobs is None else dprobs.float().clone()
    if dweights is not None:
        dw = dweights.float()
        if renorm:
            raw = probs.gather(1, idx)
            s = raw.sum(-1, keepdim=True) + 1e-20
            dw = (dw - (dw * weights).sum(-1, keepdim=True)) / s
        total.scatter_add_(1, idx, dw)
    return probs * (total - (probs * total).sum(-1, keepdim=True))


def moe_sort(experts, num_experts, align=1):
    """Sort of the T*k (token, slot) pairs by expert id into per-expert segments padded to `align` rows.

    Returns (token_of [Mp]: source token of every sorted row, -1 in pad rows; pos [T, k]: sorted row of
    every pair; offsets [E+1]: segment boundaries).  On CUDA the segments are padded to 128 rows (one GEMM
    tile) whatever `align` says; index tensors are int32 there and int64 on CPU."""
    if experts.is_cuda:
        r = N.moe_sort(experts, num_experts, align)
        if r is not NotImplemented:
            return r
        _fell("moe_sort")
    return _moe_sort_torch(experts, num_experts, align)


def moe_sort_unpadded(experts, num_experts):
    """Dense (unpadded) expert sort, used where rows travel between ranks before they are grouped."""
    if experts.is_cuda:
        r = N.moe_sort(experts, num_experts, 0)
        if r is not NotImplemented:
            return r
        _fell("moe_sort_unpadded")
    return _moe_sort_torch(experts, num_experts, 1)


def _moe_sort_torch(experts, num_experts, align):
    T, k = experts.shape
    flat = experts.reshape(-1).long()
    perm = torch.sort(flat, stable=True)[1]
    counts = torch.bincount(flat, minlength=num_experts)
    padded = (counts + align - 1) // align * align
    offsets = torch.zeros(num_experts + 1, dtype=torch.int64, device=experts.device)
    offsets[1:] = torch.cumsum(padded, 0)
    starts = torch.zeros(num_experts, dtype=torch.int64, device=experts.device)
    starts[1:] = torch.cumsum(counts, 0)[:-1]
    sorted_e = flat[perm]
    dest = offsets[:-1][sorted_e] + (torch.arange(perm.numel(), device=experts.device) - starts[sorted_e])
    total = int(offsets[-1]) if align > 1 else perm.numel()
    token_of = torch.full((total,), -1, dtype=torch.int64, device=experts.device)
    token_of[dest] = perm // k
    pos = torch.empty(T * k, dtype=torch.int64, device=experts.device)
    pos[perm] = dest
    return token_of, pos.reshape(T, k), offsets


def gather_rows(x, rows):
    """x[rows] for a 2-D x; negative row ids give zero rows."""
    if x.is_cuda:
        r = N.gather_rows(x, rows)
        if r is not NotImplemented:
            return r
        _fell("gather_rows")
    rl = rows.long()
    out = x.index_select(0, rl.clamp_min(0))
    neg = rl < 0
    if bool(neg.any()):
        out[neg] = 0
    return out


def scatter_add_rows(src, rows, num_rows, out_dtype=None):
    """out[rows[i]] += src[i] (rows with a negative id are skipped), fp32 accumulate."""
    if src.is_cuda:
        r = N.scatter_add_rows(src, rows, num_rows, out_dtype)
        if r is not NotImplemented:
            return r
        _fell("scatter_add_rows")
    out = torch.zeros(num_rows, src.shape[1], dtype=torch.float32, device=src.device)
    rl = rows.long()
    keep = rl >= 0
    out.index_add_(0, rl[keep], src.float()[keep])
    return out.to(out_dtype or src.dtype)


def moe_combine(y, w, pos):
    """out[t] = sum_j w[t, j] * y[pos[t, j]]."""
    if y.is_cuda:
        r = N.moe_combine(y, w, pos)
        if r is not NotImplemented:
            return r
        _fell("moe_combine")
    T, k = w.shape
    rows = y.index_select(0, pos.reshape(-1).long()).reshape(T, k, -1)
    return (rows.float() * w.float().unsqueeze(-1)).sum(1).to(y.dtype)


def moe_combine_bwd(g, y, w, pos):
    """Returns (dy [like y, zero in rows no pair points to], dw [T, k] fp32)."""
    if y.is_cuda:
        r = N.moe_combine_bwd(g, y, w, pos)
        if r is not NotImplemented:
            return r
        _fell("moe_combine_bwd")
    T, k = w.shape
    idx = pos.reshape(-1).long()
    rows = y.index_select(0, idx).reshape(T, k, -1)
    dw = (rows.float() * g.float().unsqueeze(1)).sum(-1)
    dy = torch.zeros_like(y)
    dy[idx] = (g.float().unsqueeze(1) * w.float().unsqueeze(-1)).to(y.dtype).reshape(T * k, -1)
    return dy, dw


def _seg(offsets):
    o = offsets.tolist()
    return [(e, o[e], o[e + 1]) for e in range(len(o) - 1) if o[e + 1] > o[e]]


def grouped_linear(x, w, offsets, out=None):
    """y[s:e] = x[s:e] @ w[g].T for each group g with rows offsets[g]:offsets[g+1]. x [M,K], w [G,N,K].
    `out`: optional [M, N] contiguous buffer of x's dtype that receives y."""
    if x.is_cuda:
        r = N.grouped_linear(x, w, offsets, out)
        if r is not NotImplemented:
            return r
        _fell("grouped_linear")
    y = torch.zeros(x.shape[0], w.shape[1], dtype=x.dtype, device=x.device)
    for g, s, e in _seg(offsets):
        y[s:e] = x[s:e] @ w[g].t()
    if out is not None:
        out.copy_(y)
        return out
    return y


def grouped_dgrad(gy, w, offsets):
    """dx[s:e] = gy[s:e] @ w[g]. gy [M,N], w [G,N,K]."""
    if gy.is_cuda:
        r = N.grouped_dgrad(gy, w, offsets)
        if r is not NotImplemented:
            return r
        _fell("grouped_dgrad")
    dx = torch.zeros(gy.shape[0], w.shape[2], dtype=gy.dtype, device=gy.device)
    for g, s, e in _seg(offsets):
        dx[s:e] = gy[s:e] @ w[g]
    return dx


def grouped_wgrad(gy, x, offsets, num_groups, out_dtype=None):
    """dw[g] = gy[s:e].T @ x[s:e] (fp32 accumulate). Returns [G,N,K]."""
    if gy.is_cuda:
        r = N.grouped_wgrad(gy, x, offsets, num_groups, out_dtype)
        if r is not NotImplemented:
            return r
        _fell("grouped_wgrad")
    dw = torch.zeros(num_groups, gy.shape[1], x.shape[1], dtype=torch.float32, device=gy.device)
    for g, s, e in _seg(offsets):
        dw[g] = gy[s:e].float().t() @ x[s:e].float()
    return dw.to(out_dtype or gy.dtype)


# =============================== sort / select / index producers ================================
def _last_dim_call(t, dim, fn):
    """Runs `fn` on `t` with `dim` moved last (contiguous) and moves the result dims back."""
    d = dim % t.dim() if t.dim() else 0
    moved = t if d == t.dim() - 1 else t.movedim(d, -1)
    out = fn(contiguous(moved))
    if out is NotImplemented:
        return out
    if d == t.dim() - 1:
        return out
    return tuple(o.movedim(-1, d) for o in out) if isinstance(out, tuple) else out.movedim(-1, d)


def sort(t, dim=-1, descending=False):
    """Stable sort -> (values, int64 indices)."""
    if _cuda(t) and t.dim() > 0:
        out = _last_dim_call(t, dim, lambda x: N.sort_rows(x, x.shape[-1], descending))
        if out is not NotImplemented:
            return out
    _fb(t, "sort")
    return tuple(torch.sort(t, dim=dim, descending=descending, stable=True))


def topk(t, k, dim=-1, largest=True):
    if _cuda(t) and t.dim() > 0:
        out = _last_dim_call(t, dim, lambda x: N.sort_rows(x, k, largest))
        if out is not NotImplemented:
            return out
    _fb(t, "topk")
    return tuple(torch.topk(t, k, dim=dim, largest=largest, sorted=True))


def argmax(t, dim=None, keepdim=False, is_min=False):
    if _cuda(t) and t.numel() > 0:
        if dim is None:
            out = N.argmax_rows(contiguous(t).reshape(-1), is_min)
            if out is not NotImplemented:
                return out.reshape([1] * t.dim()) if keepdim else out.reshape(())
        else:
            d = dim % t.dim()
            moved = t if d == t.dim() - 1 else t.movedim(d, -1)
            out = N.argmax_rows(contiguous(moved), is_min)
            if out is not NotImplemented:
                return out.unsqueeze(d) if keepdim else out
    _fb(t, "argmax")
    fn = torch.argmin if is_min else torch.argmax
    return fn(t, dim=dim, keepdim=keepdim)


def bincount(idx, weights=None, minlength=0):
    flat = idx.reshape(-1)
    if _cuda(flat) and flat.numel() > 0 and flat.dtype in (torch.int32, torch.int64):
        nbins = max(int(flat.max().item()) + 1, int(minlength))
        w = None if weights is None else weights.reshape(-1)
        if w is None or w.dtype == torch.float32:
            out = N.bincount(contiguous(flat), None if w is None else contiguous(w), nbins)
            if out is not NotImplemented:
                return out
    _fb(flat, "bincount")
    return torch.bincount(flat.long(), weights=None if weights is None else weights.reshape(-1), minlength=minlength)


def nonzero(t):
    """[count, ndim] int64 coordinates, row-major order."""
    if _cuda(t) and t.numel() > 0:
        flat = N.nonzero_flat(contiguous(t))
        if flat is not NotImplemented:
            if t.dim() <= 1:
                return flat.reshape(-1, max(t.dim(), 0)) if t.dim() == 0 else flat.reshape(-1, 1)
            coords = []
            rem = flat
            for size in reversed(t.shape):
                coords.append(rem % size)
                rem = torch.div(rem, size, rounding_mode="floor")
            return torch.stack(coords[::-1], dim=1)
    _fb(t, "nonzero")
    return torch.nonzero(t)


def triu_tril(t, diag, upper):
    if _cuda(t) and t.dim() >= 2:
        out = N.triu_tril(contiguous(t), diag, upper)
        if out is not NotImplemented:
            return out
    _fb(t, "triu_tril")
    return torch.triu(t, diagonal=diag) if upper else torch.tril(t, diagonal=diag)


def one_hot(idx, classes, dtype=torch.int64):
    if _cuda(idx):
        out = N.one_hot(idx.contiguous(), classes, dtype)
        if out is not NotImplemented:
            return out
    _fb(idx, "one_hot")
    return torch.nn.functional.one_hot(idx.long(), classes).to(dtype)


def arange(start, end, step, dtype, device):
    dev = torch.device(device)
    n = max(0, -(-(end - start) // step)) if all(isinstance(v, int) for v in (start, end, step)) \
        else max(0, int(math.ceil((end - start) / step)))
    if dev.type == "cuda" and N.available() and n > 0:
        out = N.arange(start, step, n, dtype, dev)
        if out is not NotImplemented:
            return out
    if dev.type == "cuda" and n > 0:
        _fell("arange")
    return torch.arange(start, end, step, dtype=dtype, device=dev)


def repeat_interleave(t, repeats, dim=None):
    if _cuda(t) and isinstance(repeats, int) and t.numel() > 0:
        src, d = (t.reshape(-1), 0) if dim is None else (t, dim)
        out = N.repeat_interleave(src.contiguous(), repeats, d)
        if out is not NotImplemented:
            return out
    _fb(t, "repeat_interleave")
    return torch.repeat_interleave(t, repeats, dim=dim)


# ================================== indexing engine ==============================
def cat(tensors, dim=0):
    tensors = list(tensors)
    if tensors and tensors[0].is_cuda:
        live = [t for t in tensors if not (t.dim() == 1 and t.numel() == 0)]     # torch skips legacy empty tensors
        if live and all(t.is_cuda and t.dtype == live[0].dtype for t in live):
            out = N.cat([contiguous(t) for t in live], dim)
            if out is not NotImplemented:
                return out
        _fell("cat")
    return torch.cat(tensors, dim)


def stack(tensors, dim=0):
    tensors = list(tensors)
    if tensors and tensors[0].is_cuda and all(t.shape == tensors[0].shape for t in tensors):
        d = dim % (tensors[0].dim() + 1)
        out = cat([t.unsqueeze(d) for t in tensors], d)
        return out
    return torch.stack(tensors, dim)


def _index_tensor(index, device):
    if index.device != device:
        index = index.to(device)
    return index if index.dtype in (torch.int32, torch.int64) else index.long()


def gather(a, dim, index):
    if a.is_cuda:
        out = N.gather_dim(a, dim, _index_tensor(index, a.device))
        if out is not NotImplemented:
            return out
        _fell("gather")
    return torch.gather(a, dim, index.long())


def scatter(a, dim, index, src, add=False):
    """Out of place: a copy of `a` with `src` (tensor or scalar) scattered (or scatter-added) along `dim`."""
    if a.is_cuda:
        out = clone(a)
        s = src
        if isinstance(s, torch.Tensor) and s.dtype != a.dtype:
            s = to_dtype(s, a.dtype)
        r = N.scatter_dim_(out, dim, _index_tensor(index, a.device), s, add)
        if r is not NotImplemented:
            return out
        _fell("scatter_add" if add else "scatter")
    if add:
        return a.scatter_add(dim, index.long(), src)
    return a.scatter(dim, index.long(), src)


def scatter_(a, dim, index, src):
    """In place `a.scatter_(dim, index, src)`."""
    if a.is_cuda:
        s = src
        if isinstance(s, torch.Tensor) and s.dtype != a.dtype:
            s = to_dtype(s, a.dtype)
        if N.scatter_dim_(a, dim, _index_tensor(index, a.device), s, False) is not NotImplemented:
            return a
        _fell("scatter")
    return a.scatter_(dim, index.long(), src)


def scatter_add_into_zeros(shape, dim, index, src):
    """zeros(shape).scatter_add_(dim, index, src): the gradient of `gather` / `topk`."""
    if src.is_cuda:
        out = torch.empty(shape, dtype=src.dtype, device=src.device)
        zero_(out)
        r = N.scatter_dim_(out, dim, _index_tensor(index, src.device), src, True)
        if r is not NotImplemented:
            return out
        _fell("scatter_add")
    out = torch.zeros(shape, dtype=src.dtype, device=src.device)
    return out.scatter_add_(dim, index.long(), src)


def getitem(a, index):
    if a.is_cuda:
        from . import indexing
        out = indexing.getitem(a, index)
        if out is not NotImplemented:
            return out
        _fell("getitem")
    return a[index]


def setitem_(a, index, value):
    """`a[index] = value` in place."""
    if a.is_cuda:
        from . import indexing
        if indexing.setitem_(a, index, value) is not NotImplemented:
            return a
        _fell("setitem")
    a[index] = value
    return a


def getitem_backward(shape, index, g):
    if g.is_cuda:
        from . import indexing
        out = indexing.getitem_backward(shape, index, g)
        if out is not NotImplemented:
            return out
        _fell("getitem_backward")
    out = torch.zeros(shape, dtype=g.dtype, device=g.device)
    items = index if isinstance(index, tuple) else (index,)
    if not any(isinstance(i, (torch.Tensor, list)) for i in items):
        out[index] = g
    elif all(isinstance(i, torch.Tensor) for i in items):
        out.index_put_(tuple(i if i.dtype == torch.bool else i.long() for i in items), g, accumulate=True)
    else:
        lin = torch.arange(out.numel(), device=out.device).reshape(out.shape)[index]
        out.reshape(-1).index_add_(0, lin.reshape(-1), g.reshape(-1).to(out.dtype))
    return out


def index_add_rows_(acc, rows, idx):
    """acc[idx[i], :] += rows[i, :] in place for any float accumulator dtype (atomic adds).  False: not available."""
    if not acc.is_cuda:
        return False
    flat = idx.reshape(-1)
    r2 = rows.reshape(-1, acc.shape[1])
    if r2.dtype != acc.dtype:
        r2 = to_dtype(r2, acc.dtype)
    r2 = contiguous(r2)
    flat = flat if flat.dtype in (torch.int32, torch.int64) else flat.long()
    r = N.index_put_(acc, [0], [contiguous(flat)], (flat.numel(),), [], [1], r2, add=True)
    return r is not NotImplemented


def zeros(shape, dtype, device):
    out = torch.empty(shape, dtype=dtype, device=device)
    return zero_(out) if out.is_cuda else out.zero_()
