"""Mixture-of-experts decoder family.

API parity: reference `genesis/models/transformers/moe.py` — `MoEGate` (`:40-148`),
`MoEExpert` (`:151-191`), `AddAuxiliaryLoss` (`:194-216`), `MoELayer` (`:219-401`),
`MoEAttention` (`:464-632`), `MoEDecoderLayer` (`:635-761`), `DenseFFN` (`:764-812`),
`MoEPreTrainedModel` (`:815-904`), `MoEModel` (`:907-1005`), `MoEForCausalLM`
(`:1008-1157`), with the same state-dict keys (`mlp.gate.weight`,
`mlp.experts.{e}.{gate,up,down}_proj.weight`, top-level `lm_head.weight`).

Execution differs completely.  The reference loops over all experts in Python with a
boolean-mask gather per expert (one device→host readback each) and unsorts with two
`argsort`s; here a layer is: router kernel (softmax + top-k + renormalise + per-expert
counts) → one stable sort of the (token, slot) pairs by expert → row gather → grouped
SwiGLU GEMMs over the ragged expert segments → weighted scatter back.  Expert weights are
stored stacked `[E, I, H]` (exposed per expert in the state dict), which is what the
grouped GEMM and expert-parallel sharding consume.  With an expert-parallel group the
dispatch/combine steps become all-to-alls (`genesis_b200.parallel.ep`).
"""
import math

import torch

from ... import init, nn
from ...function import Function, AMPPolicy
from ...nn import functional as F
from ...nn.modules.module import Module, Parameter
from ...ops import dispatch as K
from .sampling import sample_next
from ...tensor import Tensor
from ...amp_state import amp_state
from .components import RotaryEmbedding, apply_rope
from .config import MoEConfig, get_moe_config


# ------------------------------------------------------------------------------------
# router
# ------------------------------------------------------------------------------------
class RouterFunction(Function):
    """logits [T, E] -> (topk weights [T, k] fp32, probabilities [T, E] fp32); the selected
    expert ids and per-expert counts are returned through `ctx_out` (not differentiable)."""
    raw = True
    amp_policy = AMPPolicy.FP32

    @staticmethod
    def forward(ctx, logits, k, renorm, aux):
        w, e, probs, counts = K.moe_router(logits, k, renorm)
        ctx.save_for_backward(probs, e, w)
        ctx.renorm = renorm
        aux["experts"], aux["counts"] = e, counts
        return w, probs

    @staticmethod
    def backward(ctx, dw, dprobs):
        probs, e, w = ctx.saved_tensors
        return K.moe_router_bwd(dw, dprobs, probs, e, w, ctx.renorm)


class AddAuxiliaryLoss(Function):
    """Identity on `x` that makes `loss` part of the graph with gradient 1."""
    raw = True
    amp_policy = AMPPolicy.PRESERVE

    @staticmethod
    def forward(ctx, x, loss):
        ctx.meta = (loss.dtype, loss.shape, loss.device)
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        dt, shape, dev = ctx.meta
        return g, torch.ones(shape, dtype=dt, device=dev)


class MoEGate(Module):
    def __init__(self, hidden_size, num_experts, top_k, aux_loss_alpha=0.01, seq_aux=True,
                 norm_topk_prob=True, scoring_func="softmax"):
        super().__init__()
        self.hidden_size, self.num_experts, self.top_k = hidden_size, num_experts, top_k
        self.aux_loss_alpha, self.seq_aux = aux_loss_alpha, seq_aux
        self.norm_topk_prob, self.scoring_func = norm_topk_prob, scoring_func
        self.weight = Parameter(init.randn(num_experts, hidden_size, std=0.02))

    def route(self, hidden_states):
        """Returns (indices [T,k] raw int32 torch tensor, weights Tensor [T,k], probs Tensor [T,E], counts)."""
        if self.scoring_func != "softmax":
            raise NotImplementedError(f"Unsupported scoring function: {self.scoring_func}")
        H = hidden_states.shape[-1]
        flat = F.reshape(hidden_states, (-1, H))
        logits = F.linear(flat, self.weight)
        aux = {}
        w, probs = RouterFunction.apply(logits, self.top_k, self.top_k > 1 and self.norm_topk_prob, aux)
        return aux["experts"], w, probs, aux["counts"]

    def forward(self, hidden_states):
        B, S = hidden_states.shape[0], hidden_states.shape[1]
        idx, w, probs, counts = self.route(hidden_states)
        aux_loss = None
        if self.training and self.aux_loss_alpha > 0.0:
            aux_loss = self._compute_auxiliary_loss(probs, idx, B, S)
        return Tensor._wrap(idx.long()), w, aux_loss

    def _compute_auxiliary_loss(self, scores, topk_indices, batch_size, seq_len):
        E, k = self.num_experts, self.top_k
        idx = topk_indices if isinstance(topk_indices, torch.Tensor) else topk_indices._t
        if self.seq_aux:
            ce = torch.zeros(batch_size, E, dtype=torch.float32, device=idx.device)
            ce.scatter_add_(1, idx.reshape(batch_size, -1).long(),
                            torch.ones(batch_size, seq_len * k, dtype=torch.float32, device=idx.device))
            ce = ce / (seq_len * k / E)
            mean_scores = F.mean(F.reshape(scores, (batch_size, seq_len, E)), axis=1)
            return F.mean(F.sum(Tensor._wrap(ce) * mean_scores, axis=1)) * self.aux_loss_alpha
        ce = torch.bincount(idx.reshape(-1).long(), minlength=E).float() / idx.numel()
        pi = F.mean(scores, axis=0)
        return F.sum(pi * Tensor._wrap(ce * E)) * self.aux_loss_alpha


# ------------------------------------------------------------------------------------
# experts
# ------------------------------------------------------------------------------------
def _swiglu_mlp(mod, x):
    """down(silu(gate(x)) * up(x)) with the gate and up projections as one GEMM over the stacked weights."""
    biases = [mod.gate_proj.bias, mod.up_proj.bias] if mod.gate_proj.bias is not None else None
    return mod.down_proj(F.swiglu_fused(F.fused_linear(x, [mod.gate_proj.weight, mod.up_proj.weight], biases)))


class MoEExpert(Module):
    """One SwiGLU expert: down(silu(gate(x)) * up(x))."""

    def __init__(self, hidden_size, intermediate_size, bias=False):
        super().__init__()
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size
        self.silu = nn.SiLU()
        self.gate_proj = nn.Linear(hidden_size, intermediate_size, bias=bias)
        self.up_proj = nn.Linear(hidden_size, intermediate_size, bias=bias)
        self.down_proj = nn.Linear(intermediate_size, hidden_size, bias=bias)

    def forward(self, x):
        return _swiglu_mlp(self, x)


class _ExpertView:
    """`experts[e]`: callable view of one expert of a `GroupedExperts` stack."""

    def __init__(self, owner, e):
        self.owner, self.e = owner, e

    def __call__(self, x):
        o, e = self.owner, self.e
        I = o.intermediate_size
        g = F.linear(x, o.w_gate_up[e][:I])
        u = F.linear(x, o.w_gate_up[e][I:])
        return F.linear(F.swiglu(g, u), o.w_down[e])


class GroupedExpertsFunction(Function):
    """Sorted rows through their expert's SwiGLU MLP via grouped GEMMs.
    x [M, H] (rows sorted by expert), offsets [E+1]; weights stacked per expert: wgu [E, 2 I, H] (gate rows, then up
    rows) and wd [E, H, I].  Two grouped GEMMs and one activation pass forward; four grouped GEMMs and one activation
    pass backward (down weight gradient, down data gradient, gate|up weight gradient, gate|up data gradient).
    `out`: optional buffer for y (the expert-parallel transport hands in its symmetric staging buffer, so the
    outputs need no copy before the peers pull them)."""
    raw = True
    amp_policy = AMPPolicy.PRESERVE

    @staticmethod
    def forward(ctx, x, wgu, wd, offsets, compute_dtype, out=None):
        master = wgu.dtype
        if compute_dtype is not None:
            x = K.to_dtype(x, compute_dtype)
            wgu_c, wd_c = (F._cached_param_cast(w, compute_dtype) for w in (wgu, wd))
        else:
            wgu_c, wd_c = wgu, wd
        gu = K.grouped_linear(x, wgu_c, offsets)
        h = K.swiglu_fused_fwd(gu)
        y = K.grouped_linear(h, wd_c, offsets, out=out)
        ctx.save_for_backward(x, gu, h, wgu_c, wd_c, offsets)
        ctx.master = master
        return y

    @staticmethod
    def backward(ctx, gy):
        x, gu, h, wgu, wd, offsets = ctx.saved_tensors
        E = wgu.shape[0]
        gy = K.to_dtype(gy, x.dtype) if gy.dtype != x.dtype else gy
        gy = gy if gy.is_contiguous() else K.contiguous(gy)
        dwd = K.grouped_wgrad(gy, h, offsets, E, ctx.master)
        dh = K.grouped_dgrad(gy, wd, offsets)
        dgu = K.swiglu_fused_bwd(dh, gu)
        dwgu = K.grouped_wgrad(dgu, x, offsets, E, ctx.master)
        dx = K.grouped_dgrad(dgu, wgu, offsets)
        return dx, dwgu, dwd


class DispatchFunction(Function):
    """Row gather into expert-sorted order: out[i] = x[token_of[i]]; backward scatter-adds."""
    raw = True
    amp_policy = AMPPolicy.PRESERVE

    @staticmethod
    def forward(ctx, x, token_of):
        ctx.save_for_backward(token_of)
        ctx.n = x.shape[0]
        return K.gather_rows(x, token_of)

    @staticmethod
    def backward(ctx, g):
        (token_of,) = ctx.saved_tensors
        return K.scatter_add_rows(g, token_of, ctx.n, g.dtype)


class CombineFunction(Function):
    """out[t] = sum_j w[t, j] * y[pos[t, j]] where pos maps (token, slot) to its sorted row."""
    raw = True
    amp_policy = AMPPolicy.PRESERVE

    @staticmethod
    def forward(ctx, y, w, pos):
        ctx.save_for_backward(y, w, pos)
        return K.moe_combine(y, w, pos)

    @staticmethod
    def backward(ctx, g):
        y, w, pos = ctx.saved_tensors
        g = g if g.dtype == y.dtype else K.to_dtype(g, y.dtype)
        dy, dw = K.moe_combine_bwd(g if g.is_contiguous() else K.contiguous(g), y, w, pos)
        return dy, dw.to(w.dtype)


class GroupedExperts(Module):
    """All experts of a layer as two stacked parameters (optionally only a shard of them): `w_gate_up`
    [E, 2 I, H] holds every expert's gate rows followed by its up rows, so both projections are one grouped GEMM;
    `w_down` [E, H, I].  `w_gate` / `w_up` are views for reading; the state dict keeps per-expert
    `{e}.gate_proj / up_proj / down_proj.weight` entries."""

    def __init__(self, num_experts, hidden_size, intermediate_size, first_expert=0, total_experts=None):
        super().__init__()
        self.num_experts, self.hidden_size, self.intermediate_size = num_experts, hidden_size, intermediate_size
        self.first_expert = first_expert
        self.total_experts = total_experts if total_experts is not None else num_experts
        self.w_gate_up = Parameter(init.randn(num_experts, 2 * intermediate_size, hidden_size, std=0.02))
        self.w_down = Parameter(init.randn(num_experts, hidden_size, intermediate_size, std=0.02))

    @property
    def w_gate(self):
        return Tensor._wrap(self.w_gate_up._t[:, :self.intermediate_size])

    @property
    def w_up(self):
        return Tensor._wrap(self.w_gate_up._t[:, self.intermediate_size:])

    def __len__(self):
        return self.num_experts

    def __getitem__(self, e):
        return _ExpertView(self, e)

    def __iter__(self):
        return (self[e] for e in range(self.num_experts))

    def forward(self, x_sorted, offsets, out=None):
        cd = amp_state.dtype if amp_state.enabled else None
        return GroupedExpertsFunction.apply(x_sorted, self.w_gate_up, self.w_down,
                                            Tensor._wrap(offsets) if isinstance(offsets, torch.Tensor) else offsets,
                                            cd, out)

    # state dict: experts.{e}.{gate,up,down}_proj.weight, e = global expert id
    def _state_dict_hook(self, sd, prefix):
        I = self.intermediate_size
        gu = sd.pop(prefix + "w_gate_up")
        down = sd.pop(prefix + "w_down")
        for e in range(self.num_experts):
            base = f"{prefix}{self.first_expert + e}."
            sd[base + "gate_proj.weight"] = Tensor._wrap(gu._t[e, :I])
            sd[base + "up_proj.weight"] = Tensor._wrap(gu._t[e, I:])
            sd[base + "down_proj.weight"] = Tensor._wrap(down._t[e])

    def _load_state_dict_pre_hook(self, sd, prefix):
        def take(name):
            keys = [f"{prefix}{self.first_expert + e}.{name}.weight" for e in range(self.num_experts)]
            if not all(k in sd for k in keys):
                return None
            parts = [sd.pop(k) for k in keys]
            return torch.stack([p._t if isinstance(p, Tensor) else torch.as_tensor(p) for p in parts])
        # (older checkpoints of this framework: stacked w_gate / w_up entries)
        g = sd.pop(prefix + "w_gate")._t if prefix + "w_gate" in sd else take("gate_proj")
        u = sd.pop(prefix + "w_up")._t if prefix + "w_up" in sd else take("up_proj")
        if g is not None and u is not None:
            sd[prefix + "w_gate_up"] = Tensor._wrap(torch.cat((g, u), dim=1))
        d = take("down_proj")
        if d is not None:
            sd[prefix + "w_down"] = Tensor._wrap(d)


class MoELayer(Module):
    def __init__(self, hidden_size, num_experts, top_k, intermediate_size, num_shared_experts=None,
                 shared_intermediate_size=None, aux_loss_alpha=0.01, seq_aux=True, norm_topk_prob=True,
                 expert_bias=False, ep_group=None):
        super().__init__()
        self.hidden_size, self.num_experts, self.top_k = hidden_size, num_experts, top_k
        self.num_shared_experts = num_shared_experts
        self.gate = MoEGate(hidden_size, num_experts, top_k, aux_loss_alpha, seq_aux, norm_topk_prob)
        self.ep = ep_group
        if ep_group is not None and ep_group.size > 1:
            local = num_experts // ep_group.size
            self.experts = GroupedExperts(local, hidden_size, intermediate_size,
                                          first_expert=ep_group.rank * local, total_experts=num_experts)
        else:
            self.experts = GroupedExperts(num_experts, hidden_size, intermediate_size)
        if num_shared_experts is not None and num_shared_experts > 0:
            if shared_intermediate_size is None:
                shared_intermediate_size = intermediate_size * num_shared_experts
            self.shared_experts = MoEExpert(hidden_size, shared_intermediate_size, bias=expert_bias)
        else:
            self.shared_experts = None

    def forward(self, hidden_states):
        shape = hidden_states.shape
        B, S = shape[0], shape[1]
        idx, w, probs, counts = self.gate.route(hidden_states)
        aux_loss = None
        if self.training and self.gate.aux_loss_alpha > 0.0:
            aux_loss = self.gate._compute_auxiliary_loss(probs, idx, B, S)
        x = F.reshape(hidden_states, (-1, self.hidden_size))
        if self.ep is not None and self.ep.size > 1:
            from ...parallel.ep import expert_parallel_forward
            out = expert_parallel_forward(self, x, idx, w)
        else:
            out = self._local_forward(x, idx, w)
        out = F.reshape(out, shape)
        if aux_loss is not None:
            out = AddAuxiliaryLoss.apply(out, aux_loss)
        if self.shared_experts is not None:
            out = out + self.shared_experts(hidden_states)
        return out

    def _local_forward(self, x, idx, w):
        token_of, pos, offsets = K.moe_sort(idx, self.num_experts)
        xs = DispatchFunction.apply(x, Tensor._wrap(token_of))
        ys = self.experts(xs, offsets)
        return CombineFunction.apply(ys, w, Tensor._wrap(pos))


# ------------------------------------------------------------------------------------
# decoder
# ------------------------------------------------------------------------------------
class MoEAttention(Module):
    """GQA self-attention with the HF-style signature (`past_key_value`, `use_cache`)."""

    def __init__(self, config, layer_idx=None):
        super().__init__()
        self.config, self.layer_idx = config, layer_idx
        self.hidden_size = config.hidden_size
        self.num_heads = config.num_attention_heads
        self.num_key_value_heads = config.num_key_value_heads
        self.head_dim = config.head_dim
        self.num_key_value_groups = self.num_heads // self.num_key_value_heads
        b = config.attention_bias
        self.q_proj = nn.Linear(self.hidden_size, self.num_heads * self.head_dim, bias=b)
        self.k_proj = nn.Linear(self.hidden_size, self.num_key_value_heads * self.head_dim, bias=b)
        self.v_proj = nn.Linear(self.hidden_size, self.num_key_value_heads * self.head_dim, bias=b)
        self.o_proj = nn.Linear(self.num_heads * self.head_dim, self.hidden_size, bias=b)
        self.rotary_emb = RotaryEmbedding(self.head_dim, max_position_embeddings=config.max_position_embeddings,
                                          base=config.rope_theta)

    def forward(self, hidden_states, attention_mask=None, position_ids=None, past_key_value=None,
                use_cache=False):
        B, S, _ = hidden_states.shape
        past = 0 if past_key_value is None else past_key_value[0].shape[1]
        if position_ids is None and past > 0:
            position_ids = Tensor._wrap(torch.arange(past, past + S, device=hidden_states._t.device).expand(B, S).contiguous())
        # q, k and v projections as one GEMM over the stacked weights; RoPE reads its head slices in place
        biases = [self.q_proj.bias, self.k_proj.bias, self.v_proj.bias] if self.q_proj.bias is not None else None
        y = F.fused_linear(hidden_states, [self.q_proj.weight, self.k_proj.weight, self.v_proj.weight], biases)
        rot = self.rotary_emb
        need = S + past if position_ids is None else S + past
        if need > rot.max_seq_len_cached:
            rot._build(need)
        q, k, v = F.qkv_rope(y, rot.cos_cached, rot.sin_cached, position_ids, self.num_heads,
                             self.num_key_value_heads, self.head_dim)
        if past_key_value is not None:
            k = F.cat((past_key_value[0], k), dim=1)
            v = F.cat((past_key_value[1], v), dim=1)
        present = (k, v) if use_cache else None
        if attention_mask is None:
            o = F.flash_attention(q, k, v, causal=True)
        else:
            qt, kt, vt = (F.transpose(t, 1, 2) for t in (q, k, v))
            if self.num_key_value_groups > 1:
                kt = F.repeat_interleave(kt, self.num_key_value_groups, dim=1)
                vt = F.repeat_interleave(vt, self.num_key_value_groups, dim=1)
            s = (qt @ F.transpose(kt, -1, -2)) * (1.0 / math.sqrt(self.head_dim)) + attention_mask
            o = F.transpose(F.softmax(s, dim=-1) @ vt, 1, 2)
        o = F.reshape(o, (B, S, self.num_heads * self.head_dim))
        return self.o_proj(o), present

    def _repeat_kv(self, hidden_states, n_rep):
        return hidden_states if n_rep == 1 else F.repeat_interleave(hidden_states, n_rep, dim=1)


class DenseFFN(Module):
    def __init__(self, hidden_size, intermediate_size, hidden_act="silu", bias=False):
        super().__init__()
        self.gate_proj = nn.Linear(hidden_size, intermediate_size, bias=bias)
        self.up_proj = nn.Linear(hidden_size, intermediate_size, bias=bias)
        self.down_proj = nn.Linear(intermediate_size, hidden_size, bias=bias)
        self.hidden_act = hidden_act

    def forward(self, x):
        if self.hidden_act == "silu":
            return _swiglu_mlp(self, x)
        act = {"gelu": F.gelu, "relu": F.relu}[self.hidden_act]
        return self.down_proj(act(self.gate_proj(x)) * self.up_proj(x))


class MoEDecoderLayer(Module):
    def __init__(self, config, layer_idx, ep_group=None):
        super().__init__()
        self.hidden_size, self.layer_idx = config.hidden_size, layer_idx
        self.self_attn = MoEAttention(config, layer_idx)
        self.is_moe_layer = self._is_moe_layer(layer_idx, config)
        if self.is_moe_layer:
            self.mlp = MoELayer(config.hidden_size, config.num_local_experts, config.num_experts_per_tok,
                                config.moe_intermediate_size, config.num_shared_experts,
                                config.shared_expert_intermediate_size, config.router_aux_loss_coef,
                                config.seq_aux, config.norm_topk_prob, config.expert_bias, ep_group=ep_group)
        else:
            self.mlp = self._build_dense_mlp(config)
        self.input_layernorm = nn.RMSNorm(config.hidden_size, eps=config.norm_eps)
        self.post_attention_layernorm = nn.RMSNorm(config.hidden_size, eps=config.norm_eps)

    def _is_moe_layer(self, layer_idx, config):
        if config.use_moe_in_all_layers:
            return True
        if layer_idx < config.first_moe_layer:
            return False
        return (layer_idx - config.first_moe_layer) % config.moe_layer_interval == 0

    def _build_dense_mlp(self, config):
        return DenseFFN(config.hidden_size, config.intermediate_size, config.hidden_act, config.mlp_bias)

    def forward(self, hidden_states, attention_mask=None, position_ids=None, past_key_value=None,
                use_cache=False):
        a, present = self.self_attn(self.input_layernorm(hidden_states), attention_mask, position_ids,
                                    past_key_value, use_cache)
        h = hidden_states + a
        return h + self.mlp(self.post_attention_layernorm(h)), present

    def forward_deferred(self, stream, branch, attention_mask=None, position_ids=None, past_key_value=None,
                         use_cache=False):
        """The same layer with its residual additions folded into the normalisations (one fused kernel each way):
        its input is `stream + branch` (`branch` None for the first layer); returns (stream', branch', present)
        with stream' + branch' the layer's output."""
        x, n = self.input_layernorm.add_forward(stream, branch)
        a, present = self.self_attn(n, attention_mask, position_ids, past_key_value, use_cache)
        h, n2 = self.post_attention_layernorm.add_forward(x, a)
        return h, self.mlp(n2), present


class MoEPreTrainedModel(Module):
    def __init__(self, config):
        super().__init__()
        self.config = config

    def _init_weights(self, module):
        std = self.config.initializer_range
        if isinstance(module, (nn.Linear, nn.Embedding, MoEGate)):
            w = module.weight
            w._t.copy_(init.randn(*w.shape, std=std, device=w.device, dtype=w.dtype)._t)
            if getattr(module, "bias", None) is not None:
                module.bias._t.zero_()
        elif isinstance(module, GroupedExperts):
            for attr, _ in GroupedExperts._NAMES:
                w = getattr(module, attr)
                w._t.copy_(init.randn(*w.shape, std=std, device=w.device, dtype=w.dtype)._t)

    def post_init(self):
        self.apply(self._init_weights)


class MoEModel(MoEPreTrainedModel):
    def __init__(self, config, ep_group=None):
        super().__init__(config)
        self.vocab_size = config.vocab_size
        self.embed_tokens = nn.Embedding(config.vocab_size, config.hidden_size)
        self.layers = nn.ModuleList([MoEDecoderLayer(config, i, ep_group) for i in range(config.num_hidden_layers)])
        self.norm = nn.RMSNorm(config.hidden_size, eps=config.norm_eps)

    def forward(self, input_ids, attention_mask=None, position_ids=None, past_key_values=None, use_cache=None):
        use_cache = bool(use_cache)
        h = self.embed_tokens(input_ids)
        mask4 = None
        if attention_mask is not None:
            B, S = input_ids.shape
            am = attention_mask._t if isinstance(attention_mask, Tensor) else attention_mask
            causal = torch.full((S, S), float("-inf"), device=am.device).triu(1)
            pad = torch.zeros(B, 1, 1, S, device=am.device).masked_fill(am.reshape(B, 1, 1, S) == 0, float("-inf"))
            mask4 = Tensor._wrap(causal.reshape(1, 1, S, S) + pad)
        presents = [] if use_cache else None
        branch = None
        for i, layer in enumerate(self.layers):
            past = past_key_values[i] if past_key_values is not None else None
            h, branch, present = layer.forward_deferred(h, branch, mask4, position_ids, past, use_cache)
            if use_cache:
                presents.append(present)
        return self.norm.add_forward(h, branch)[1], presents


class MoEForCausalLM(MoEPreTrainedModel):
    def __init__(self, config, ep_group=None):
        super().__init__(config)
        self.model = MoEModel(config, ep_group)
        self.vocab_size = config.vocab_size
        self.lm_head = nn.Linear(config.hidden_size, config.vocab_size, bias=False)
        if config.tie_word_embeddings:
            self.lm_head.weight = self.model.embed_tokens.weight

    def forward(self, input_ids, attention_mask=None, position_ids=None, past_key_values=None, use_cache=None,
                labels=None, return_logits=True):
        """Logits, or `(loss, logits)` when `labels` are given (labels are shifted by one here,
        as in the reference). `return_logits=False` returns only the loss and lets the fused
        cross-entropy reuse the logits buffer for their gradient."""
        h, _ = self.model(input_ids, attention_mask, position_ids, past_key_values, use_cache)
        logits = self.lm_head(h)
        if labels is None:
            return logits
        B, S, V = logits.shape
        lab = labels._t if isinstance(labels, Tensor) else labels
        shifted = torch.full_like(lab, -100)
        shifted[..., :-1] = lab[..., 1:]
        loss = F.cross_entropy(F.reshape(logits, (-1, V)), Tensor._wrap(shifted.reshape(-1)), ignore_index=-100,
                               _inplace_backward=not return_logits)
        return (loss, logits) if return_logits else loss

    @classmethod
    def from_pretrained(cls, config_or_path):
        config = get_moe_config(config_or_path) if isinstance(config_or_path, str) else config_or_path
        return cls(config)

    def generate(self, input_ids, max_new_tokens=100, temperature=1.0, top_k=None, top_p=None):
        from ... import grad_mode
        self.eval()
        generated = input_ids
        with grad_mode.no_grad():
            for _ in range(max_new_tokens):
                logits = self(generated)
                tok = sample_next(logits._t[:, -1, :], temperature, top_k, top_p)
                generated = Tensor._wrap(torch.cat((generated._t, tok.to(generated._t.dtype)), dim=1))
        return generated


class MoETransformerBlock(MoEDecoderLayer):
    """Legacy name kept for the reference's older entry point (`moe.py:404-456`)."""

    def forward(self, x, *a, **k):
        out = super().forward(x, *a, **k)
        return out[0]
