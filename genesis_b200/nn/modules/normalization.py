"""Normalisation layers. Parity: reference `genesis/nn/modules/normalization.py:12-137`."""
from ... import init
from .. import functional as F
from .module import Module, Parameter


class BatchNorm1d(Module):
    def __init__(self, dim, eps=1e-5, momentum=0.1, device=None, dtype="float32"):
        super().__init__()
        self.dim, self.eps, self.momentum = dim, eps, momentum
        self.weight = Parameter(init.ones(dim, device=device, dtype=dtype))
        self.bias = Parameter(init.zeros(dim, device=device, dtype=dtype))
        self.running_mean = init.zeros(dim, device=device, dtype=dtype)
        self.running_var = init.ones(dim, device=device, dtype=dtype)

    def forward(self, x):
        if self.training:
            n = x.shape[0]
            mean = F.sum(x, axis=0, keepdims=True) / n
            centered = x - mean
            var = F.sum(centered * centered, axis=0, keepdims=True) / n
            m = self.momentum
            self.running_mean._t = (m * mean._t.reshape(-1) + (1 - m) * self.running_mean._t).detach()
            self.running_var._t = (m * var._t.reshape(-1) + (1 - m) * self.running_var._t).detach()
            xn = centered / F.sqrt(var + self.eps)
        else:
            xn = (x - self.running_mean) / F.sqrt(self.running_var + self.eps)
        return self.weight * xn + self.bias


class LayerNorm(Module):
    def __init__(self, dim, eps=1e-5, device=None, dtype="float32"):
        super().__init__()
        self.dim, self.eps = dim, eps
        self.weight = Parameter(init.ones(dim, device=device, dtype=dtype))
        self.bias = Parameter(init.zeros(dim, device=device, dtype=dtype))

    def forward(self, x):
        return F.layer_norm(x, self.weight, self.bias, self.eps)


class FusedLayerNorm(LayerNorm):
    def __init__(self, dim, eps=1e-6, device=None, dtype="float32"):
        super().__init__(dim, eps, device, dtype)


class RMSNorm(Module):
    """y = x / sqrt(mean(x^2) + eps) * weight, one fused kernel each way, float32 math."""

    def __init__(self, dim, eps=1e-6, device=None, dtype="float32"):
        super().__init__()
        self.dim, self.eps = dim, eps
        self.weight = Parameter(init.ones(dim, device=device, dtype=dtype))

    def forward(self, x):
        return F.rms_norm(x, self.weight, self.eps)

    def add_forward(self, x, residual=None):
        """(x + residual, self(x + residual)) from one fused kernel; with `residual=None` simply (x, self(x)).
        Lets a pre-norm block hand its branch output to the next normalisation instead of adding it itself."""
        if residual is None:
            return x, self.forward(x)
        return F.add_rms_norm(x, residual, self.weight, self.eps)
