"""`Linear`, `Flatten`. Parity: reference `genesis/nn/modules/linear.py:10-51`."""
from ... import init
from .. import functional as F
from .module import Module, Parameter


class Linear(Module):
    """y = x W^T + b, weight [out, in] ~ N(0, 0.02), bias zeros."""

    def __init__(self, in_features, out_features, bias=True, device=None, dtype="float32"):
        super().__init__()
        self.in_features = in_features
        self.out_features = out_features
        self.weight = Parameter(init.randn(out_features, in_features, std=0.02, device=device, dtype=dtype))
        self.bias = Parameter(init.zeros(out_features, device=device, dtype=dtype)) if bias else None

    def forward(self, x):
        return F.linear(x, self.weight, self.bias)

    def extra_repr(self):
        return f"in_features={self.in_features}, out_features={self.out_features}, bias={self.bias is not None}"


class Flatten(Module):
    def forward(self, x):
        return F.reshape(x, (x.shape[0], -1))
