"""Rotary embedding helpers. Parity: reference `genesis/models/transformers/components.py:30-179`.

`RotaryEmbedding` keeps `[max_pos, dim]` cos/sin caches (halves duplicated, i.e.
`cat(freqs, freqs)`), registered as non-persistent buffers, extended on demand.
`apply_rotary_pos_emb` keeps the reference signature on `[B, H, S, D]` tensors;
`apply_rope` is the fused path on `[B, S, H, D]` (one kernel per tensor instead of ~14).
"""
import numpy as np

from ...tensor import Tensor, tensor
from ... import nn
from ...nn import functional as F

# The reference selects a PyTorch re-implementation of these classes with NANOCHAT_BACKEND=torch; here there is one
# implementation, and the name stays for code that reads it.
BACKEND = "genesis"



def find_multiple(n, k):
    return n if n % k == 0 else n + k - (n % k)


def rotate_half(x):
    d = x.shape[-1] // 2
    return F.cat((-x[..., d:], x[..., :d]), dim=-1)


class RotaryEmbedding(nn.Module):
    def __init__(self, dim, max_position_embeddings=2048, base=10000.0, device=None):
        super().__init__()
        self.dim, self.base = dim, float(base)
        self.max_position_embeddings = max_position_embeddings
        self._device = device
        self._build(max_position_embeddings)

    def _build(self, seq_len):
        inv = 1.0 / (self.base ** (np.arange(0, self.dim, 2, dtype=np.float64) / self.dim))
        t = np.arange(seq_len, dtype=np.float64)
        freqs = np.outer(t, inv)
        emb = np.concatenate([freqs, freqs], axis=-1)
        dev = self._device
        old = self.__dict__.get("cos_cached")
        if old is not None:
            dev = old.device
        self.max_seq_len_cached = seq_len
        self.register_buffer("inv_freq", tensor(inv.astype(np.float32), device=dev), persistent=False)
        self.register_buffer("cos_cached", tensor(np.cos(emb).astype(np.float32), device=dev), persistent=False)
        self.register_buffer("sin_cached", tensor(np.sin(emb).astype(np.float32), device=dev), persistent=False)

    def forward(self, x=None, seq_len=None):
        if seq_len is not None and seq_len > self.max_seq_len_cached:
            self._build(seq_len)
        if seq_len is None:
            return self.cos_cached, self.sin_cached
        return self.cos_cached[:seq_len], self.sin_cached[:seq_len]


def apply_rotary_pos_emb(q, k, cos, sin, position_ids=None):
    """q, k: [B, H, S, D]; cos, sin: [S or max_pos, D]; position_ids: [B, S] or None."""
    if position_ids is not None:
        cos = F.unsqueeze(cos[position_ids], 1)
        sin = F.unsqueeze(sin[position_ids], 1)
    else:
        S = q.shape[-2]
        cos = F.reshape(cos[:S], (1, 1, S, cos.shape[-1]))
        sin = F.reshape(sin[:S], (1, 1, S, sin.shape[-1]))
    q_embed = q * cos + rotate_half(q) * sin
    k_embed = k * cos + rotate_half(k) * sin
    return q_embed, k_embed


def apply_rope(x, rotary, position_ids=None):
    """Fused rotate-half RoPE on x [B, S, H, D]."""
    S = x.shape[1]
    if S > rotary.max_seq_len_cached:
        rotary._build(S)
    pos = None if position_ids is None else position_ids
    return F.rope(x, rotary.cos_cached, rotary.sin_cached, pos)
