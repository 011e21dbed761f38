"""Activation modules. Parity: reference `genesis/nn/modules/activation.py:10-70`."""
from .. import functional as F
from .module import Module


class ReLU(Module):
    def forward(self, x):
        return F.relu(x)


class Softmax(Module):
    def __init__(self, dim=-1):
        super().__init__()
        self.dim = dim

    def forward(self, x):
        return F.softmax(x, dim=self.dim)


class SiLU(Module):
    def forward(self, x):
        return F.silu(x)


class GELU(Module):
    def forward(self, x):
        return F.gelu(x)


class Sigmoid(Module):
    def forward(self, x):
        return F.sigmoid(x)


class Tanh(Module):
    def forward(self, x):
        return F.tanh(x)


class Residual(Module):
    def __init__(self, fn):
        super().__init__()
        self.fn = fn

    def forward(self, x):
        return self.fn(x) + x
