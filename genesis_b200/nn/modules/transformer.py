"""Attention / feed-forward building blocks.
Parity: reference `genesis/nn/modules/transformer.py:15-105`."""
import math

from ... import init
from ...functional import triu
from .. import functional as F
from .activation import SiLU, Softmax
from .dropout import Dropout
from .linear import Linear
from .module import Module, Parameter


class FeedFowardSwiGLU(Module):
    """down(silu(gate(x)) * up(x)) followed by Dropout(0.1). (Class name spelled as in the reference.)"""

    def __init__(self, dim, hidden_dim):
        super().__init__()
        self.gate = Linear(dim, hidden_dim, bias=False)
        self.down = Linear(hidden_dim, dim, bias=False)
        self.up = Linear(dim, hidden_dim, bias=False)
        self.act = SiLU()
        self.dropout = Dropout(0.1)

    def forward(self, x):
        return self.dropout(self.down(F.swiglu(self.gate(x), self.up(x))))


FeedForwardSwiGLU = FeedFowardSwiGLU


def _split_heads(x, w_qkv, dim, heads):
    B, S = x.shape[0], x.shape[1]
    qkv = F.reshape(x @ w_qkv, (B, S, 3, heads, dim // heads))
    q, k, v = (F.reshape(t, (B, S, heads, dim // heads)) for t in F.split(qkv, dim=2))
    return q, k, v


class MultiheadAttention(Module):
    """Causal self-attention with explicit softmax; returns (output, attention probabilities)."""

    def __init__(self, dim=64, heads=1, device=None, dtype="float32"):
        super().__init__()
        self.dim, self.heads = dim, heads
        self.w_qkv = Parameter(init.kaiming_uniform(dim, dim * 3, device=device, dtype=dtype))
        self.w_out = Parameter(init.kaiming_uniform(dim, dim, device=device, dtype=dtype))
        self.softmax = Softmax()

    def forward(self, x):
        B, S = x.shape[0], x.shape[1]
        q, k, v = (F.transpose(t, 1, 2) for t in _split_heads(x, self.w_qkv, self.dim, self.heads))
        mask = triu(init.full((S, S), float("-inf"), device=x.device), k=1)
        att = self.softmax(q @ F.transpose(k, -1, -2) / math.sqrt(self.dim // self.heads) + mask)
        out = F.reshape(F.transpose(att @ v, 1, 2), (B, S, self.dim)) @ self.w_out
        return out, att


class FusedMultiheadAttention(Module):
    """Same projections, flash-attention kernel for the core; returns (output, None)."""

    def __init__(self, dim=64, heads=1, device=None, dtype="float32"):
        super().__init__()
        self.dim, self.heads = dim, heads
        self.w_qkv = Parameter(init.kaiming_uniform(dim, dim * 3, device=device, dtype=dtype))
        self.w_out = Parameter(init.kaiming_uniform(dim, dim, device=device, dtype=dtype))

    def forward(self, x):
        B, S = x.shape[0], x.shape[1]
        q, k, v = (F.contiguous(t) for t in _split_heads(x, self.w_qkv, self.dim, self.heads))
        o = F.flash_attention(q, k, v, causal=True)
        return F.reshape(o, (B, S, self.dim)) @ self.w_out, None
