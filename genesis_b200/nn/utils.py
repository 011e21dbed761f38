"""`clip_grad_norm_`. Parity: reference `genesis/nn/utils.py:10-31`; here the squared norm of
all gradients is accumulated on the device by one multi-tensor kernel and the scale is
applied without a per-parameter Python loop of reductions."""
import torch

from ..ops import dispatch as K


def norm(data, p=2):
    """p-norm of all elements as a differentiable 0-d tensor (reference `nn/utils.py:3-7`: (sum x**p)**(1/p), no
    absolute value)."""
    from .. import nn as _nn
    F = _nn.functional
    return F.pow_scalar(F.summation(F.pow_scalar(data, p)), 1.0 / p) if hasattr(F, "pow_scalar") else \
        (data ** p).sum() ** (1.0 / p)


def clip_grad_norm_(parameters, max_norm, norm_type=2, sync=True):
    """Scale all gradients so that their total norm is at most `max_norm`; returns the norm before clipping.

    `sync=False` (CUDA, 2-norm) keeps everything on the device: the coefficient min(1, max_norm / (norm + 1e-6)) is
    computed by device arithmetic, applied by one multi-tensor kernel, and the norm comes back as a 0-d `Tensor`;
    no host read, so the call can sit inside a captured CUDA graph.  The default reads the norm back as a float
    (the reference's return type) and skips the scaling pass when nothing has to be clipped."""
    from ..tensor import Tensor
    if isinstance(parameters, Tensor):
        parameters = [parameters]
    params = [p for p in parameters if p.grad is not None]
    if not params:
        return 0.0
    for j in {id(f): f for f in (getattr(p, "_late_join", None) for p in params) if f is not None}.values():
        j()                                   # a data-parallel wrapper left a bucket all-reduce in flight: wait for it
    grads = [p.grad._t for p in params]
    if norm_type == 2:
        acc = torch.zeros(1, dtype=torch.float32, device=grads[0].device)
        K.grad_norm_sq(grads, acc)
        if not sync and grads[0].is_cuda:
            total_t = acc.sqrt()
            K.scale_grads_(grads, (max_norm / (total_t + 1e-6)).clamp_(max=1.0))
            return Tensor._wrap(total_t.reshape(()))
        total = float(acc.sqrt().item())
    elif norm_type == float("inf"):
        total = max(float(g.abs().max()) for g in grads)
    else:
        total = sum(float(g.float().abs().pow(norm_type).sum()) for g in grads) ** (1.0 / norm_type)
    coef = max_norm / (total + 1e-6)
    if coef < 1:
        K.scale_grads_(grads, coef)
    return total


def fused_parameter_groups(model):
    """Parameter lists that layers of `model` multiply as one stacked matrix: the q/k/v projections of every attention
    block and the gate/up projections of every SwiGLU block (weights, and biases where present).  Hand them to
    `Optimizer.enable_shadows(dtype, groups=...)` so that the low-precision copies of each list live in one buffer."""
    groups = []
    for m in model.modules():
        for names in (("q_proj", "k_proj", "v_proj"), ("gate_proj", "up_proj")):
            subs = [getattr(m, n, None) for n in names]
            if any(s is None or getattr(s, "weight", None) is None for s in subs):
                continue
            groups.append([s.weight for s in subs])
            if all(getattr(s, "bias", None) is not None for s in subs):
                groups.append([s.bias for s in subs])
    return groups
