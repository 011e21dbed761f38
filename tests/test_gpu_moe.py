"""Mixture-of-experts kernels on the GPU: expert sort into padded segments, grouped GEMMs (forward,
dgrad, wgrad over ragged segments), combine, and a whole MoE layer / model against the CPU path."""
import numpy as np
import pytest
import torch

import genesis_b200 as genesis
from genesis_b200.ops import dispatch as K
from genesis_b200.ops import native as N

pytestmark = pytest.mark.gpu
DEV = "cuda"


def rnd(*shape, dt=torch.float32, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed + sum(shape))
    return (torch.randn(*shape, generator=g) * scale).to(dt)


@pytest.mark.parametrize("T,E,k", [(64, 8, 2), (1000, 128, 8), (300, 16, 4), (5, 4, 1)])
def test_sort_and_grouped_gemms(T, E, k):
    g = torch.Generator().manual_seed(T)
    experts = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)]).to(torch.int32).to(DEV)
    token_of, pos, offsets = K.moe_sort(experts, E)
    off = offsets.cpu().tolist()
    assert off[0] == 0 and all(o % 128 == 0 for o in off) and token_of.numel() >= off[-1]
    tk, ps = token_of.cpu().long(), pos.cpu().long()
    for t in range(0, T, max(1, T // 7)):
        for j in range(k):
            r = int(ps[t, j])
            e = int(experts[t, j])
            assert off[e] <= r < off[e + 1] and int(tk[r]) == t
    counts = torch.bincount(experts.reshape(-1).long().cpu(), minlength=E)
    assert int((tk >= 0).sum()) == T * k
    for e in range(E):
        assert int((tk[off[e]:off[e + 1]] >= 0).sum()) == int(counts[e])
    H, I = 64, 96
    x = rnd(T, H, dt=torch.bfloat16).to(DEV)
    xs = K.gather_rows(x, token_of)
    assert float(xs[tk < 0].abs().sum()) == 0.0
    w = rnd(E, I, H, dt=torch.bfloat16, seed=1, scale=0.2).to(DEV)
    y = K.grouped_linear(xs, w, offsets)
    N.check_status()
    rows_e = torch.zeros(token_of.numel(), dtype=torch.long)
    for e in range(E):
        rows_e[off[e]:off[e + 1]] = e
    ref = torch.einsum("mk,mnk->mn", xs.float().cpu(), w.float().cpu()[rows_e])
    valid = torch.arange(token_of.numel()) < off[-1]
    torch.testing.assert_close(y.float().cpu()[valid], ref[valid], atol=3e-2, rtol=3e-2)
    gy = rnd(token_of.numel(), I, dt=torch.bfloat16, seed=2).to(DEV)
    gy[tk.to(DEV) < 0] = 0
    dx = K.grouped_dgrad(gy, w, offsets)
    refdx = torch.einsum("mn,mnk->mk", gy.float().cpu(), w.float().cpu()[rows_e])
    torch.testing.assert_close(dx.float().cpu()[valid], refdx[valid], atol=5e-2, rtol=3e-2)
    dw = K.grouped_wgrad(gy, xs, offsets, E, torch.float32)
    N.check_status()
    refdw = torch.zeros(E, I, H)
    for e in range(E):
        refdw[e] = gy.float().cpu()[off[e]:off[e + 1]].t() @ xs.float().cpu()[off[e]:off[e + 1]]
    torch.testing.assert_close(dw.cpu(), refdw, atol=5e-2, rtol=3e-2)
    wts = torch.rand(T, k, generator=g).to(DEV)
    out = K.moe_combine(y, wts, pos)
    refo = (y.float().cpu()[ps.reshape(-1)].reshape(T, k, I) * wts.cpu().unsqueeze(-1)).sum(1)
    torch.testing.assert_close(out.float().cpu(), refo, atol=3e-2, rtol=3e-2)
    gout = rnd(T, I, dt=torch.bfloat16, seed=5).to(DEV)
    dy, dwt = K.moe_combine_bwd(gout, y, wts, pos)
    rdy, rdw = K.moe_combine_bwd(gout.float().cpu(), y.float().cpu(), wts.cpu(), ps)
    torch.testing.assert_close(dy.float().cpu(), rdy, atol=3e-2, rtol=3e-2)
    torch.testing.assert_close(dwt.cpu(), rdw, atol=0.2, rtol=5e-2)


def test_moe_layer_and_model_match_cpu():
    from genesis_b200.models.transformers import MoEConfig, MoEForCausalLM
    cfg = MoEConfig(vocab_size=256, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=2,
                    num_key_value_heads=1, head_dim=64, num_local_experts=8, num_experts_per_tok=2,
                    moe_intermediate_size=64, max_position_embeddings=128, router_aux_loss_coef=0.01)
    torch.manual_seed(3)
    genesis.manual_seed(3)
    cpu = MoEForCausalLM(cfg)
    gpu = MoEForCausalLM(cfg)
    gpu.load_state_dict(cpu.state_dict())
    gpu.cuda()
    ids = torch.randint(0, 256, (2, 128), generator=torch.Generator().manual_seed(1))
    lc, _ = cpu(genesis.Tensor(ids), labels=genesis.Tensor(ids))
    lc.backward()
    with genesis.amp.autocast(dtype=genesis.bfloat16):
        lg, _ = gpu(genesis.Tensor(ids.cuda()), labels=genesis.Tensor(ids.cuda()))
    lg.backward()
    N.check_status()
    assert abs(lc.item() - lg.item()) < 5e-2, (lc.item(), lg.item())
    gc = dict(cpu.named_parameters())
    bad = []
    for name, p in gpu.named_parameters():
        assert p.grad is not None, name
        a, b = p.grad._t.float().cpu(), gc[name].grad._t
        err = float((a - b).norm() / (b.norm() + 1e-6))
        if err > 0.15:
            bad.append((name, err))
    assert not bad, bad
    opt = genesis.optim.AdamW(gpu.parameters(), lr=1e-3)
    opt.step()
