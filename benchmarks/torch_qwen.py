"""The same Qwen-shaped decoder in plain PyTorch (cuBLAS GEMMs, `scaled_dot_product_attention`, torch's fused AdamW,
`torch.nn.parallel.DistributedDataParallel` over NCCL): the context arm of `bench.py --impl torch`.

It is what the reference's own benchmark suite compares itself with (a torch restatement of the model,
`benchmark/bench_qwen.py:35-41, 288, 384`); it is not the reference and is never reported as such.
"""
import math

import torch
import torch.nn as nn
import torch.nn.functional as F


class RMSNorm(nn.Module):
    def __init__(self, dim, eps):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.eps = eps

    def forward(self, x):
        return F.rms_norm(x, (x.shape[-1],), self.weight, self.eps)


def rope_tables(head_dim, max_pos, theta, device):
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, device=device, dtype=torch.float32) / head_dim))
    t = torch.arange(max_pos, device=device, dtype=torch.float32)
    f = torch.outer(t, inv)
    emb = torch.cat((f, f), dim=-1)
    return emb.cos(), emb.sin()


def apply_rope(x, cos, sin):
    # x: [B, H, S, D]
    d = x.shape[-1] // 2
    rot = torch.cat((-x[..., d:], x[..., :d]), dim=-1)
    return x * cos + rot * sin


class Block(nn.Module):
    def __init__(self, c):
        super().__init__()
        H, D = c["hidden_size"], c["head_dim"]
        self.hq, self.hkv, self.d = c["num_attention_heads"], c["num_key_value_heads"], D
        self.q_proj = nn.Linear(H, self.hq * D, bias=True)
        self.k_proj = nn.Linear(H, self.hkv * D, bias=True)
        self.v_proj = nn.Linear(H, self.hkv * D, bias=True)
        self.o_proj = nn.Linear(self.hq * D, H, bias=False)
        self.gate_proj = nn.Linear(H, c["intermediate_size"], bias=False)
        self.up_proj = nn.Linear(H, c["intermediate_size"], bias=False)
        self.down_proj = nn.Linear(c["intermediate_size"], H, bias=False)
        self.input_layernorm = RMSNorm(H, c["norm_eps"])
        self.post_attention_layernorm = RMSNorm(H, c["norm_eps"])

    def forward(self, x, cos, sin):
        B, S, _ = x.shape
        h = self.input_layernorm(x)
        q = self.q_proj(h).view(B, S, self.hq, self.d).transpose(1, 2)
        k = self.k_proj(h).view(B, S, self.hkv, self.d).transpose(1, 2)
        v = self.v_proj(h).view(B, S, self.hkv, self.d).transpose(1, 2)
        q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
        o = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)
        x = x + self.o_proj(o.transpose(1, 2).reshape(B, S, self.hq * self.d))
        h = self.post_attention_layernorm(x)
        return x + self.down_proj(F.silu(self.gate_proj(h)) * self.up_proj(h))


class TorchQwen(nn.Module):
    def __init__(self, c):
        super().__init__()
        self.c = c
        self.embed_tokens = nn.Embedding(c["vocab_size"], c["hidden_size"])
        self.layers = nn.ModuleList([Block(c) for _ in range(c["num_hidden_layers"])])
        self.norm = RMSNorm(c["hidden_size"], c["norm_eps"])
        for m in self.modules():
            if isinstance(m, (nn.Linear, nn.Embedding)):
                nn.init.normal_(m.weight, 0.0, 0.02)
                if getattr(m, "bias", None) is not None:
                    nn.init.zeros_(m.bias)
        self._rope = None

    def forward(self, idx, labels):
        B, S = idx.shape
        if self._rope is None or self._rope[0].shape[0] < S:
            cos, sin = rope_tables(self.c["head_dim"], max(S, self.c["max_position_embeddings"]), self.c["rope_theta"],
                                   idx.device)
            self._rope = (cos, sin)
        cos, sin = self._rope[0][:S].to(torch.bfloat16), self._rope[1][:S].to(torch.bfloat16)
        x = self.embed_tokens(idx)
        for layer in self.layers:
            x = layer(x, cos, sin)
        logits = F.linear(self.norm(x), self.embed_tokens.weight)          # tied output projection
        return F.cross_entropy(logits.view(-1, logits.shape[-1]).float(), labels)
