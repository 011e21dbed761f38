"""Model families on CPU: module tree and state-dict keys, weight tying, loss/backward, checkpoint round trip,
sampling and generation (dense Qwen and MoE)."""
import numpy as np
import torch

import genesis_b200 as genesis
from genesis_b200.models.transformers import (TransformerConfig, MoEConfig, QwenForCausalLM, MoEForCausalLM,
                                              get_moe_config, get_transformer_config)
from genesis_b200.models.transformers.sampling import sample_next


def _dense_cfg(**kw):
    base = dict(vocab_size=97, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                num_key_value_heads=2, head_dim=16, max_position_embeddings=64, rope_theta=1e4, norm_eps=1e-6)
    base.update(kw)
    return TransformerConfig(**base)


def _moe_cfg(**kw):
    base = dict(vocab_size=89, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4,
                num_key_value_heads=2, head_dim=8, max_position_embeddings=64, num_experts_per_tok=2,
                num_local_experts=4, moe_intermediate_size=48, router_aux_loss_coef=0.01)
    base.update(kw)
    return MoEConfig(**base)


def test_dense_state_dict_keys_and_tying():
    genesis.manual_seed(0)
    m = QwenForCausalLM(_dense_cfg(tie_word_embeddings=True, attention_bias=True))
    keys = set(m.state_dict().keys())
    for k in ("model.embed_tokens.weight", "model.norm.weight", "model.layers.0.self_attn.q_proj.weight",
              "model.layers.0.self_attn.q_proj.bias", "model.layers.1.self_attn.o_proj.weight",
              "model.layers.0.mlp.gate_proj.weight", "model.layers.0.mlp.down_proj.weight",
              "model.layers.1.input_layernorm.weight", "model.layers.1.post_attention_layernorm.weight"):
        assert k in keys, k
    assert "model.layers.0.self_attn.o_proj.bias" not in keys
    assert m.model.lm_head.weight is m.model.embed_tokens.weight
    n_unique = len({id(p) for p in m.parameters()})
    assert n_unique == len(list(m.parameters()))                   # the shared weight is listed once
    untied = QwenForCausalLM(_dense_cfg(tie_word_embeddings=False))
    assert untied.model.lm_head.weight is not untied.model.embed_tokens.weight


def test_dense_loss_backward_and_checkpoint_roundtrip(tmp_path):
    genesis.manual_seed(1)
    cfg = _dense_cfg(tie_word_embeddings=True)
    m = QwenForCausalLM(cfg)
    idx = genesis.Tensor(torch.randint(0, cfg.vocab_size, (2, 12)))
    labels = genesis.Tensor(torch.randint(0, cfg.vocab_size, (24,)))
    loss, logits = m(idx, labels=labels)
    assert logits.shape == (2, 12, cfg.vocab_size)
    assert abs(float(loss.item()) - np.log(cfg.vocab_size)) < 1.0
    loss.backward()
    g = m.model.embed_tokens.weight.grad
    assert g is not None and float(g._t.abs().sum()) > 0          # embedding + lm_head contributions, one tensor
    path = tmp_path / "dense.pth"
    genesis.save(m.state_dict(), str(path))
    m2 = QwenForCausalLM(cfg)
    m2.load_state_dict(genesis.load(str(path)))
    with genesis.no_grad():
        a, b = m(idx), m2(idx)
    assert torch.equal(a._t, b._t)
    # a checkpoint written without the tied head still loads
    sd = {k: v for k, v in m.state_dict().items() if k != "model.lm_head.weight"}
    QwenForCausalLM(cfg).load_state_dict(sd)
    assert get_transformer_config("qwen2.5-0.5b").hidden_size == 896


def test_causality_of_the_dense_model():
    genesis.manual_seed(2)
    m = QwenForCausalLM(_dense_cfg())
    m.eval()
    a = torch.randint(0, 97, (1, 10))
    b = a.clone()
    b[0, 7:] = (b[0, 7:] + 1) % 97
    with genesis.no_grad():
        la, lb = m(genesis.Tensor(a))._t, m(genesis.Tensor(b))._t
    assert torch.allclose(la[:, :7], lb[:, :7], atol=1e-5)
    assert not torch.allclose(la[:, 7:], lb[:, 7:], atol=1e-5)


def test_dense_generate_greedy_is_deterministic_and_extends():
    genesis.manual_seed(3)
    m = QwenForCausalLM(_dense_cfg())
    prompt = genesis.Tensor(torch.randint(0, 97, (2, 5)))
    o1 = m.generate(prompt, max_new_tokens=4, temperature=0.0)
    o2 = m.generate(prompt, max_new_tokens=4, temperature=0.0)
    assert o1.shape == (2, 9) and torch.equal(o1._t, o2._t) and torch.equal(o1._t[:, :5], prompt._t)
    o3 = m.generate(prompt, max_new_tokens=3, temperature=0.8, top_k=5, top_p=0.9)
    assert o3.shape == (2, 8) and int(o3._t.max()) < 97


def test_sample_next_respects_top_k_and_top_p():
    genesis.manual_seed(4)
    logits = torch.tensor([[0.0, 5.0, 4.9, -3.0, 1.0]]).repeat(64, 1)
    assert torch.all(sample_next(logits, temperature=0.0) == 1)
    k2 = sample_next(logits, 1.0, top_k=2)
    assert set(k2.reshape(-1).tolist()) <= {1, 2} and len(set(k2.reshape(-1).tolist())) == 2
    p_small = sample_next(logits, 1.0, top_p=0.3)                  # the top token alone covers 0.3
    assert torch.all(p_small == 1)
    free = sample_next(torch.zeros(2000, 4), 1.0)
    counts = torch.bincount(free.reshape(-1), minlength=4).float() / 2000
    assert torch.all((counts - 0.25).abs() < 0.06)


def test_moe_state_dict_keys_roundtrip_and_aux_loss(tmp_path):
    genesis.manual_seed(5)
    cfg = _moe_cfg(num_shared_experts=1, shared_expert_intermediate_size=40)
    m = MoEForCausalLM(cfg)
    keys = set(m.state_dict().keys())
    for e in range(4):
        for proj in ("gate_proj", "up_proj", "down_proj"):
            assert f"model.layers.0.mlp.experts.{e}.{proj}.weight" in keys
    assert "model.layers.1.mlp.gate.weight" in keys
    assert any("shared_experts" in k for k in keys)
    idx = genesis.Tensor(torch.randint(0, cfg.vocab_size, (2, 9)))
    m.train()
    loss, logits = m(idx, labels=idx)
    assert logits.shape == (2, 9, cfg.vocab_size) and np.isfinite(float(loss.item()))
    loss.backward()
    gate_g = m.model.layers[0].mlp.gate.weight.grad
    assert gate_g is not None and float(gate_g._t.abs().sum()) > 0   # router learns through weights and aux loss
    assert float(m.model.layers[0].mlp.experts.w_down.grad._t.abs().sum()) > 0
    path = tmp_path / "moe.pth"
    genesis.save(m.state_dict(), str(path))
    m2 = MoEForCausalLM(cfg)
    m2.load_state_dict(genesis.load(str(path)))
    m.eval(), m2.eval()
    with genesis.no_grad():
        assert torch.allclose(m(idx)._t, m2(idx)._t, atol=1e-6)


def test_moe_matches_explicit_expert_loop():
    """The grouped dispatch / combine path equals the definition: every token through its top-k experts."""
    from genesis_b200.models.transformers.moe import MoELayer
    genesis.manual_seed(6)
    layer = MoELayer(16, 4, 2, 24)
    layer.eval()
    x = torch.randn(1, 7, 16)
    with genesis.no_grad():
        out = layer(genesis.Tensor(x))._t
        idx, w, _, _ = layer.gate.route(genesis.Tensor(x))
    idx_t, w_t = (idx._t if hasattr(idx, "_t") else idx), (w._t if hasattr(w, "_t") else w)
    ref = torch.zeros(7, 16)
    wg, wu, wd = layer.experts.w_gate._t, layer.experts.w_up._t, layer.experts.w_down._t
    for t in range(7):
        for j in range(2):
            e = int(idx_t.reshape(7, 2)[t, j])
            h = torch.nn.functional.silu(x[0, t] @ wg[e].t()) * (x[0, t] @ wu[e].t())
            ref[t] += float(w_t.reshape(7, 2)[t, j]) * (h @ wd[e].t())
    assert torch.allclose(out.reshape(7, 16), ref, atol=1e-5)


def test_moe_generate_and_config_validation():
    genesis.manual_seed(7)
    cfg = _moe_cfg()
    m = MoEForCausalLM(cfg)
    out = m.generate(genesis.Tensor(torch.randint(0, cfg.vocab_size, (1, 4))), max_new_tokens=3, temperature=0.0)
    assert out.shape == (1, 7)
    try:
        _moe_cfg(num_experts_per_tok=9)
        raise AssertionError("config accepted k > experts")
    except ValueError:
        pass
    assert get_moe_config("qwen3-moe-bench").num_local_experts == 128


def test_moe_kv_cache_matches_full_recompute():
    """Prefill + one cached decode step gives the hidden state of a full forward over the longer sequence (the
    fused q/k/v projection rotates the new token at its absolute position)."""
    genesis.manual_seed(11)
    m = MoEForCausalLM(_moe_cfg(attention_bias=True))
    m.eval()
    ids = torch.randint(0, 89, (2, 6))
    with genesis.no_grad():
        full, _ = m.model(genesis.Tensor(ids), None, None, None, False)
        h0, cache = m.model(genesis.Tensor(ids[:, :5]), None, None, None, True)
        h1, _ = m.model(genesis.Tensor(ids[:, 5:]), None, None, cache, True)
    assert torch.allclose(h0._t, full._t[:, :5], atol=1e-5)
    assert torch.allclose(h1._t, full._t[:, 5:], atol=1e-5)
