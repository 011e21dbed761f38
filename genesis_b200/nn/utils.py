"""`clip_grad_norm_`. Parity: reference `genesis/nn/utils.py:10-31`; here the squared norm of
all gradients is accumulated on the device by one multi-tensor kernel and the scale is
applied without a per-parameter Python loop of reductions."""
import torch

from ..ops import dispatch as K


def clip_grad_norm_(parameters, max_norm, norm_type=2):
    params = [p for p in parameters if p.grad is not None]
    if not params:
        return 0.0
    grads = [p.grad._t for p in params]
    if norm_type == 2:
        acc = torch.zeros(1, dtype=torch.float32, device=grads[0].device)
        K.grad_norm_sq(grads, acc)
        total = float(acc.sqrt().item())
    elif norm_type == float("inf"):
        total = max(float(g.abs().max()) for g in grads)
    else:
        total = sum(float(g.float().abs().pow(norm_type).sum()) for g in grads) ** (1.0 / norm_type)
    coef = max_norm / (total + 1e-6)
    if coef < 1:
        for g in grads:
            K.mul_(g, coef)
    return total
