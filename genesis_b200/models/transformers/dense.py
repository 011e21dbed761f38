"""Qwen-style dense decoder. Parity: reference `genesis/models/transformers/dense.py:30-320`
(module tree and state-dict keys: `embed_tokens`, `layers.{i}.self_attn.{q,k,v,o}_proj`,
`layers.{i}.mlp.{gate,up,down}_proj`, `layers.{i}.{input,post_attention}_layernorm`, `norm`,
`lm_head`; q/k/v projections carry a bias, o_proj does not).

What differs underneath: activations stay in `[B, S, H, D]` layout so no transpose copies
are made; RoPE is one fused kernel; attention is the GQA flash kernel (K/V are never
replicated); the MLP uses the fused SwiGLU kernel; `tie_word_embeddings=True` really shares
one Parameter between `embed_tokens` and `lm_head`; `QwenForCausalLM(idx, labels=...)` runs the
fused cross-entropy and returns `(loss, logits)`.
"""
import torch

from ... import nn
from ...nn import functional as F
from ...tensor import Tensor
from .components import RotaryEmbedding, apply_rope, find_multiple  # noqa: F401
from .config import TransformerConfig, get_transformer_config

ModelArgs = TransformerConfig

# The reference selects a PyTorch re-implementation of these classes with NANOCHAT_BACKEND=torch; here there is one
# implementation, and the name stays for code that reads it.
BACKEND = "genesis"


class Attention(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.hidden_size = config.hidden_size
        self.num_heads = config.num_attention_heads
        self.num_kv_heads = config.num_key_value_heads
        self.head_dim = config.head_dim
        self.num_key_value_groups = self.num_heads // self.num_kv_heads
        # Qwen2 always biases q/k/v (reference `dense.py:230-238`)
        self.q_proj = nn.Linear(self.hidden_size, self.num_heads * self.head_dim, bias=True)
        self.k_proj = nn.Linear(self.hidden_size, self.num_kv_heads * self.head_dim, bias=True)
        self.v_proj = nn.Linear(self.hidden_size, self.num_kv_heads * self.head_dim, bias=True)
        self.o_proj = nn.Linear(self.num_heads * self.head_dim, self.hidden_size, bias=False)
        self.rotary_emb = RotaryEmbedding(self.head_dim, max_position_embeddings=config.max_position_embeddings,
                                          base=config.rope_theta)

    def forward(self, x, position_ids=None, mask=None):
        B, S, _ = x.shape
        # q, k and v projections as one GEMM over the stacked weights; RoPE reads its head slices in place
        y = F.fused_linear(x, [self.q_proj.weight, self.k_proj.weight, self.v_proj.weight],
                           [self.q_proj.bias, self.k_proj.bias, self.v_proj.bias])
        rot = self.rotary_emb
        if S > rot.max_seq_len_cached:
            rot._build(S)
        q, k, v = F.qkv_rope(y, rot.cos_cached, rot.sin_cached, position_ids, self.num_heads, self.num_kv_heads,
                             self.head_dim)
        o = F.flash_attention(q, k, v, causal=True)
        return self.o_proj(F.reshape(o, (B, S, self.num_heads * self.head_dim)))


class FeedForward(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.gate_proj = nn.Linear(config.hidden_size, config.intermediate_size, bias=config.mlp_bias)
        self.up_proj = nn.Linear(config.hidden_size, config.intermediate_size, bias=config.mlp_bias)
        self.down_proj = nn.Linear(config.intermediate_size, config.hidden_size, bias=config.mlp_bias)
        if not config.mlp_bias:
            # the fused backward of `F.swiglu_mlp` multiplies by the [in, out] twin of this weight: ask the optimizer's
            # low-precision copies to keep one (`Optimizer.enable_shadows(transposed="auto")`)
            self.down_proj.weight.wants_transposed_copy = True

    def forward(self, x):
        # gate and up projections as one GEMM over the stacked weights; SwiGLU reads the two halves in place
        if self.gate_proj.bias is None and self.down_proj.bias is None:
            # ... and with no biases the whole MLP is one node: the activation rides in the gate|up GEMM's epilogue,
            # its gradient in the epilogue of the down projection's data-gradient GEMM
            return F.swiglu_mlp(x, self.gate_proj.weight, self.up_proj.weight, self.down_proj.weight)
        biases = [self.gate_proj.bias, self.up_proj.bias]
        return self.down_proj(F.swiglu_fused(F.fused_linear(x, [self.gate_proj.weight, self.up_proj.weight], biases)))


class TransformerBlock(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.self_attn = Attention(config)
        self.mlp = FeedForward(config)
        self.input_layernorm = nn.RMSNorm(config.hidden_size, eps=config.norm_eps)
        self.post_attention_layernorm = nn.RMSNorm(config.hidden_size, eps=config.norm_eps)

    def forward(self, x, input_pos=None, position_ids=None, mask=None):
        h = x + self.self_attn(self.input_layernorm(x), position_ids, mask)
        return h + self.mlp(self.post_attention_layernorm(h))

    def forward_deferred(self, stream, branch, position_ids=None, mask=None):
        """The same block with its residual additions folded into the normalisations: the block's input is
        `stream + branch` (`branch` None for the first block), and it returns (stream', branch') whose sum is its
        output, leaving that last addition to whoever normalises next."""
        x, n = self.input_layernorm.add_forward(stream, branch)
        h, n2 = self.post_attention_layernorm.add_forward(x, self.self_attn(n, position_ids, mask))
        return h, self.mlp(n2)


class QwenModel(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.config = config
        self.embed_tokens = nn.Embedding(config.vocab_size, config.hidden_size)
        self.layers = nn.ModuleList(TransformerBlock(config) for _ in range(config.n_layer))
        self.norm = nn.RMSNorm(config.hidden_size, eps=config.norm_eps)
        self.lm_head = nn.Linear(config.hidden_size, config.vocab_size, bias=False)
        if config.tie_word_embeddings:
            self.lm_head.weight = self.embed_tokens.weight
        self.max_batch_size = -1
        self.max_seq_length = -1

    def setup_caches(self, max_batch_size, max_seq_length):
        if self.max_seq_length >= max_seq_length and self.max_batch_size >= max_batch_size:
            return
        self.max_seq_length = find_multiple(max_seq_length, 8)
        self.max_batch_size = max_batch_size

    def hidden_states(self, idx, position_ids=None):
        x, branch = self.embed_tokens(idx), None
        for layer in self.layers:
            x, branch = layer.forward_deferred(x, branch, position_ids, None)
        return self.norm.add_forward(x, branch)[1]

    def forward(self, idx, position_ids=None):
        return self.lm_head(self.hidden_states(idx, position_ids))

    @classmethod
    def from_name(cls, name):
        return cls(get_transformer_config(name))


class QwenForCausalLM(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.config = config
        self.model = QwenModel(config)

    def forward(self, idx, labels=None, return_logits=True, **kwargs):
        """Logits `[B, S, V]`; with `labels` (already aligned with the logits, -100 = ignore)
        returns `(loss, logits)` using the fused cross-entropy.  `return_logits=False` returns
        only the loss and lets the backward pass overwrite the logits buffer with their gradient."""
        logits = self.model(idx, **kwargs)
        if labels is None:
            return logits
        V = logits.shape[-1]
        loss = F.cross_entropy(F.reshape(logits, (-1, V)), labels, ignore_index=-100,
                               _inplace_backward=not return_logits)
        return (loss, logits) if return_logits else loss

    def generate(self, input_ids, max_new_tokens=100, temperature=1.0, top_k=None, top_p=None):
        """Appends `max_new_tokens` sampled tokens to `input_ids` [B, S] (temperature 0: greedy).  The prompt is
        re-encoded every step (no KV cache in this model class, as in the reference)."""
        from ... import grad_mode
        from .sampling import sample_next
        was_training = self.training
        self.eval()
        out = input_ids
        with grad_mode.no_grad():
            for _ in range(max_new_tokens):
                logits = self(out)
                tok = sample_next(logits._t[:, -1, :], temperature, top_k, top_p)
                out = Tensor._wrap(torch.cat((out._t, tok.to(out._t.dtype)), dim=1))
        if was_training:
            self.train()
        return out

    def load_state_dict(self, state_dict, strict=True):
        sd = dict(state_dict)
        if "model.lm_head.weight" not in sd and "model.embed_tokens.weight" in sd:
            sd["model.lm_head.weight"] = sd["model.embed_tokens.weight"]
        return super().load_state_dict(sd, strict)

    @classmethod
    def from_name(cls, name):
        return cls(get_transformer_config(name))
