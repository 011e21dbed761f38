"""`Embedding`, `RotaryEmbedding`. Parity: reference `genesis/nn/modules/sparse.py:12-64`."""
import numpy as np

from ... import init
from ...tensor import Tensor, tensor
from .. import functional as F
from .module import Module, Parameter


class Embedding(Module):
    def __init__(self, num_embeddings, embedding_dim, device=None, dtype="float32"):
        super().__init__()
        self.num_embeddings, self.embedding_dim = num_embeddings, embedding_dim
        self.weight = Parameter(init.randn(num_embeddings, embedding_dim, std=0.02, device=device, dtype=dtype))

    def forward(self, x):
        return F.embedding(self.weight, x)


class RotaryEmbedding(Module):
    """cos/sin caches of shape [1, 1, max_pos, dim] (halves duplicated); `forward` returns
    the first `seq_len` positions."""

    def __init__(self, dim, max_position_embeddings=2048, base=10000):
        super().__init__()
        inv = 1.0 / (base ** (np.arange(0, dim, 2).astype(np.float32) / dim))
        t = np.arange(max_position_embeddings, dtype=np.float32)
        freqs = np.outer(t, inv)
        emb = np.concatenate([freqs, freqs], axis=-1)
        self.max_seq_len_cached = max_position_embeddings
        self.inv_freq = tensor(inv.reshape(1, -1))
        self.cos_cached = tensor(np.cos(emb).reshape(1, 1, *emb.shape))
        self.sin_cached = tensor(np.sin(emb).reshape(1, 1, *emb.shape))

    def forward(self, x, seq_len=None):
        return self.cos_cached[:, :, :seq_len, :], self.sin_cached[:, :, :seq_len, :]
