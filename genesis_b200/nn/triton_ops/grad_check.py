"""`genesis.nn.triton_ops.grad_check` of the reference: gradient unscale + finiteness check as multi-tensor kernels
(`csrc/optim.cu`).  `fused_unscale_and_check_kernel(grads, inv_scale, found_inf)` multiplies every tensor of `grads` by
`inv_scale` in place and sets the one-element float tensor `found_inf` to 1 when any value is Inf / NaN;
`check_finite_kernel(grads, found_inf)` only checks."""
from ...ops import dispatch as _K


def fused_unscale_and_check_kernel(grads, inv_scale, found_inf):
    _K.unscale_and_check([getattr(g, "_t", g) for g in grads], inv_scale, getattr(found_inf, "_t", found_inf))
    return found_inf


def check_finite_kernel(grads, found_inf):
    _K.unscale_and_check([getattr(g, "_t", g) for g in grads], None, getattr(found_inf, "_t", found_inf))
    return found_inf
