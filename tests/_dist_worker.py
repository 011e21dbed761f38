"""Worker launched by the distributed tests (one process per rank, torchrun environment).

    python -m torch.distributed.run --nproc-per-node N ... tests/_dist_worker.py --scenario S --backend gloo|nccl

Every scenario asserts on all ranks and prints `WORKER_OK <rank>` at the end.
"""
import argparse
import os
import sys

import numpy as np
import torch
import torch.distributed as tdist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import genesis_b200 as genesis  # noqa: E402
import genesis_b200.nn as nn  # noqa: E402
import genesis_b200.nn.functional as F  # noqa: E402
from genesis_b200 import distributed as dist  # noqa: E402


def dev(backend):
    return f"cuda:{torch.cuda.current_device()}" if backend == "nccl" else "cpu"


class MLP(nn.Module):
    def __init__(self, d=64, h=256, out=16):
        super().__init__()
        self.fc1 = nn.Linear(d, h)
        self.fc2 = nn.Linear(h, h)
        self.fc3 = nn.Linear(h, out)
        self.norm = nn.RMSNorm(h)

    def forward(self, x):
        return self.fc3(self.norm(F.relu(self.fc2(F.relu(self.fc1(x))))))


def scenario_collectives(a):
    r, w, d = dist.get_rank(), dist.get_world_size(), dev(a.backend)
    t = genesis.Tensor(torch.full((1000,), float(r + 1), device=d))
    dist.all_reduce(t)
    assert torch.allclose(t._t, torch.full((1000,), w * (w + 1) / 2.0, device=d))
    t = genesis.Tensor(torch.full((7,), float(r + 1), device=d))
    dist.all_reduce(t, dist.ReduceOp.MAX)
    assert float(t._t[0]) == w
    b = genesis.Tensor(torch.arange(5, dtype=torch.float32, device=d) * (r + 1))
    dist.broadcast(b, src=0)
    assert torch.equal(b._t.cpu(), torch.arange(5, dtype=torch.float32))
    outs = [genesis.Tensor(torch.zeros(3, device=d)) for _ in range(w)]
    dist.all_gather(outs, genesis.Tensor(torch.full((3,), float(r), device=d)))
    for i, o in enumerate(outs):
        assert float(o._t[0]) == i
    out = genesis.Tensor(torch.zeros(4, device=d))
    dist.reduce_scatter(out, [genesis.Tensor(torch.full((4,), float(i + r), device=d)) for i in range(w)])
    assert float(out._t[0]) == sum(r + i for i in range(w))
    inp = torch.arange(w * 2, dtype=torch.float32, device=d) + 100 * r
    res = torch.zeros(w * 2, device=d)
    dist.all_to_all_single(res, inp)
    for i in range(w):
        assert float(res[2 * i]) == 100 * i + 2 * r
    dist.barrier()
    # large, odd-sized float tensors through the default all-reduce path (peer-memory kernel on CUDA)
    for n, dt in [(1 << 20, torch.float32), (12345, torch.float32), (300001, torch.bfloat16)]:
        g = torch.Generator().manual_seed(n)
        base = torch.randn(w, n, generator=g)
        ref = base.to(dt).float().sum(0)
        x = base[r].clone().to(dt).to(d)
        dist.all_reduce(genesis.Tensor(x))
        tol = 1e-5 if dt == torch.float32 else 5e-2
        assert torch.allclose(x.float().cpu(), ref, atol=tol * w, rtol=tol), (n, dt)
    # larger / odd-sized gather, broadcast, reduce-scatter and variable-split all-to-all (on CUDA these run
    # as pull kernels over peer memory)
    for n, dt in [(70001, torch.float32), (4096, torch.bfloat16), (3, torch.int64)]:
        mine = (torch.arange(n, device=d) % 251 + 1000 * r).to(dt)
        outs = [torch.zeros(n, dtype=dt, device=d) for _ in range(w)]
        dist.all_gather([genesis.Tensor(o) for o in outs], genesis.Tensor(mine))
        for i, o in enumerate(outs):
            assert torch.equal(o, (torch.arange(n, device=d) % 251 + 1000 * i).to(dt)), (n, dt, i)
        bc = mine.clone()
        dist.broadcast(genesis.Tensor(bc), src=w - 1)
        assert torch.equal(bc, (torch.arange(n, device=d) % 251 + 1000 * (w - 1)).to(dt)), (n, dt)
    n = 30011
    ins = [torch.full((n,), float(r + 10 * i), device=d) + torch.arange(n, device=d) % 7 for i in range(w)]
    out = torch.zeros(n, device=d)
    dist.reduce_scatter(genesis.Tensor(out), [genesis.Tensor(i) for i in ins])
    ref = sum(float(q + 10 * r) for q in range(w)) + w * (torch.arange(n, device=d) % 7).float()
    assert torch.allclose(out, ref), "reduce_scatter"
    # rank r sends (d + 1 + r) rows of 24 bf16 values to rank d
    send_rows = [dd + 1 + r for dd in range(w)]
    recv_rows = [r + 1 + s_ for s_ in range(w)]
    inp = torch.cat([torch.full((send_rows[dd], 24), float(10 * r + dd), device=d) for dd in range(w)]).to(torch.bfloat16)
    res = torch.zeros(sum(recv_rows), 24, dtype=torch.bfloat16, device=d)
    dist.all_to_all_single(res, inp, recv_rows, send_rows)
    pos = 0
    for s_ in range(w):
        assert torch.all(res[pos:pos + recv_rows[s_]].float() == float(10 * s_ + r)), ("a2a", s_)
        pos += recv_rows[s_]
    dist.barrier()


def _local_grads(model_fn, x, y, seed):
    torch.manual_seed(seed)
    genesis.manual_seed(seed)
    m = model_fn()
    return m


def scenario_ddp(a):
    r, w, d = dist.get_rank(), dist.get_world_size(), dev(a.backend)
    torch.manual_seed(100 + r)           # different initial weights per rank: DDP must broadcast rank 0's
    genesis.manual_seed(100 + r)
    model = MLP().to(d)
    ref = MLP().to(d)
    ddp = nn.DistributedDataParallel(model, bucket_cap_mb=0.1)       # several buckets
    ref.load_state_dict(ddp.state_dict())
    p0 = [p._t.clone() for p in model.parameters()]
    gathered = [torch.zeros_like(p0[0]) for _ in range(w)]
    tdist.all_gather(gathered, p0[0])
    for gth in gathered:
        assert torch.equal(gth, gathered[0]), "parameters were not broadcast"
    rs = np.random.RandomState(7 + r)
    opt = genesis.optim.AdamW(ddp.parameters(), lr=1e-2)
    for step in range(3):
        x = genesis.Tensor(torch.from_numpy(rs.randn(32, 64).astype(np.float32)).to(d))
        y = genesis.Tensor(torch.from_numpy(rs.randint(0, 16, (32,))).to(d))
        # reference: local gradients of an identical un-wrapped model, averaged with the communicator
        ref.zero_grad()
        F.cross_entropy(ref(x), y).backward()
        want = []
        for p in ref.parameters():
            g = p.grad._t.clone()
            tdist.all_reduce(g)
            want.append(g / w)
        opt.zero_grad()
        F.cross_entropy(ddp(x), y).backward()
        if a.backend == "nccl":
            torch.cuda.synchronize()
            dist.symm.check_status("ddp all-reduce") if dist.symm.available() else None
        for (name, p), g in zip(model.named_parameters(), want):
            assert p.grad is not None, name
            assert torch.allclose(p.grad._t, g, atol=1e-5, rtol=1e-4), (name, step, float((p.grad._t - g).abs().max()))
        opt.step()
        ref.load_state_dict(ddp.state_dict())
    # no_sync: gradients stay local
    opt.zero_grad()
    with ddp.no_sync():
        F.cross_entropy(ddp(x), y).backward()
    g_local = model.fc1.weight.grad._t.clone()
    ref.zero_grad()
    F.cross_entropy(ref(x), y).backward()
    assert torch.allclose(g_local, ref.fc1.weight.grad._t, atol=1e-6)
    # delegation surface
    assert ddp.module is model and ddp.model is model
    assert set(ddp.state_dict()) == set(model.state_dict())
    assert ddp.fc1 is model.fc1


def scenario_ddp_tied(a):
    """Tied embedding / output weights: the parameter receives two gradient contributions per backward pass; its
    bucket must be reduced after the second one."""
    from genesis_b200.models.transformers import TransformerConfig, QwenForCausalLM
    r, w, d = dist.get_rank(), dist.get_world_size(), dev(a.backend)
    cfg = TransformerConfig(vocab_size=211, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                            num_attention_heads=4, num_key_value_heads=2, head_dim=16, max_position_embeddings=32,
                            tie_word_embeddings=True)
    genesis.manual_seed(3)
    ref = QwenForCausalLM(cfg).to(d)
    genesis.manual_seed(3)
    model = QwenForCausalLM(cfg).to(d)
    ddp = nn.DistributedDataParallel(model, bucket_cap_mb=0.05)
    rs = np.random.RandomState(100 + r)
    idx = genesis.Tensor(torch.from_numpy(rs.randint(0, 211, (2, 16))).to(d))
    lab = genesis.Tensor(torch.from_numpy(rs.randint(0, 211, (32,))).to(d))
    for step in range(2):
        for m in (ref, model):
            for p_ in m.parameters():
                p_.grad = None
        loss_ref, _ = ref(idx, labels=lab)
        loss_ref.backward()
        loss, _ = ddp(idx, labels=lab)
        loss.backward()
        if d != "cpu":
            torch.cuda.synchronize()
        for (n1, p1), (n2, p2) in zip(ref.named_parameters(), model.named_parameters()):
            g = p1.grad._t.clone()
            tdist.all_reduce(g)
            assert torch.allclose(p2.grad._t, g / w, atol=2e-5, rtol=1e-4), (step, n1, float((p2.grad._t - g / w).abs().max()))


def scenario_ddp_graph(a):
    """A data-parallel training step (forward, backward with bucket all-reduces on the communication stream, AdamW)
    replayed from a CUDA graph follows the eager data-parallel trajectory."""
    from genesis_b200.models.transformers import TransformerConfig, QwenForCausalLM
    from genesis_b200.distributed import symm
    r, d = dist.get_rank(), dev(a.backend)
    cfg = TransformerConfig(vocab_size=512, hidden_size=128, intermediate_size=256, num_hidden_layers=2,
                            num_attention_heads=2, num_key_value_heads=1, head_dim=64, max_position_embeddings=128,
                            attention_bias=True)

    def make():
        genesis.manual_seed(9)
        m = QwenForCausalLM(cfg).to(d)
        net = nn.DistributedDataParallel(m, bucket_cap_mb=0.25)
        opt = genesis.optim.AdamW(m.parameters(), lr=1e-3)

        def step(tokens):
            idx = genesis.Tensor(tokens._t[:, :-1].contiguous())
            labels = genesis.Tensor(tokens._t[:, 1:].reshape(-1).contiguous())
            with genesis.amp.autocast(dtype=genesis.bfloat16):
                loss = net(idx, labels=labels, return_logits=False)
            opt.zero_grad()
            loss.backward()
            opt.step()
            return loss
        return m, net, opt, step

    ma, neta, oa, step_a = make()
    mb, netb, ob, step_b = make()
    assert neta._use_symm and netb._use_symm
    rs = np.random.RandomState(100 + r)
    batches = [genesis.Tensor(torch.from_numpy(rs.randint(0, 512, (4, 65))).to(d)) for _ in range(6)]
    graphed = genesis.cuda.GraphedTrainStep(step_b, ob, [batches[0]], warmup=2)
    for _ in range(2):
        step_a(batches[0])
    for i, t in enumerate(batches[1:]):
        if i == 2:
            oa.lr = ob.lr = 3e-4
        la = step_a(t)
        lb = graphed(t)
        torch.cuda.synchronize()
        assert abs(float(la._t) - float(lb._t)) < 2e-3 * max(1.0, abs(float(la._t))), (i, float(la._t), float(lb._t))
    symm.check_status("graphed ddp")
    for pa, pb in zip(ma.parameters(), mb.parameters()):
        # atomics + Adam: run-to-run differences reach a few 1e-4 on average; a missed learning-rate change or
        # step count would show as 1e-3 and more, and in the losses above
        assert float((pa._t - pb._t).abs().mean()) < 6e-4
    # every rank holds the same parameters
    for pb in mb.parameters():
        g = pb._t.clone()
        tdist.broadcast(g, 0)
        assert torch.equal(g, pb._t)


def scenario_ddp_amp(a):
    """fp16-style loss scaling through DDP: an overflow on ONE rank must skip the step on ALL ranks."""
    r, w, d = dist.get_rank(), dist.get_world_size(), dev(a.backend)
    torch.manual_seed(1)
    genesis.manual_seed(1)
    model = MLP().to(d)
    scaler = genesis.amp.GradScaler(init_scale=1024.0)
    ddp = nn.DistributedDataParallel(model, grad_scaler=scaler)
    opt = genesis.optim.AdamW(ddp.parameters(), lr=1e-2)
    x = genesis.Tensor(torch.randn(8, 64).to(d))
    y = genesis.Tensor(torch.randint(0, 16, (8,)).to(d))
    before = model.fc1.weight._t.clone()
    loss = F.cross_entropy(ddp(x), y)
    if r == w - 1:
        loss = loss * float("inf")
    opt.zero_grad()
    scaler.scale(loss).backward()
    scaler.step(opt)
    assert scaler.found_inf(), "overflow flag did not reach this rank"
    scaler.update()
    assert torch.equal(model.fc1.weight._t, before), "step was not skipped"
    assert scaler.get_scale() == 512.0
    loss = F.cross_entropy(ddp(x), y)
    opt.zero_grad()
    scaler.scale(loss).backward()
    scaler.step(opt)
    scaler.update()
    assert not torch.equal(model.fc1.weight._t, before)
    chk = model.fc1.weight._t.clone()
    tdist.all_reduce(chk)
    assert torch.allclose(chk / w, model.fc1.weight._t, atol=1e-6), "ranks diverged"


def scenario_ddp_amp_clip(a):
    """DDP + GradScaler + explicit `unscale_` + gradient clipping: the gradients that reach the optimizer equal the
    mean of the ranks' true (unscaled) gradients, whether the fused all-reduce or the scaler did the unscaling."""
    r, w, d = dist.get_rank(), dist.get_world_size(), dev(a.backend)
    torch.manual_seed(2)
    genesis.manual_seed(2)
    model = MLP().to(d)
    ref = MLP().to(d)
    scaler = genesis.amp.GradScaler(init_scale=4096.0)
    ddp = nn.DistributedDataParallel(model, grad_scaler=scaler)
    ref.load_state_dict(ddp.state_dict())
    opt = genesis.optim.AdamW(ddp.parameters(), lr=1e-2)
    rs = np.random.RandomState(31 + r)
    x = genesis.Tensor(torch.from_numpy(rs.randn(16, 64).astype(np.float32)).to(d))
    y = genesis.Tensor(torch.from_numpy(rs.randint(0, 16, (16,))).to(d))
    ref.zero_grad()
    F.cross_entropy(ref(x), y).backward()
    want = []
    for p in ref.parameters():
        g = p.grad._t.clone()
        tdist.all_reduce(g)
        want.append(g / w)
    opt.zero_grad()
    scaler.scale(F.cross_entropy(ddp(x), y)).backward()
    scaler.unscale_(opt)
    for (name, p), g in zip(model.named_parameters(), want):
        assert torch.allclose(p.grad._t, g, atol=1e-5, rtol=1e-3), (name, float((p.grad._t - g).abs().max()))
    total = nn.utils.clip_grad_norm_(model.parameters(), 1e-3)
    tot = float(total.item()) if hasattr(total, "item") else float(total)
    ref_norm = float(torch.sqrt(sum((g.float() ** 2).sum() for g in want)))
    assert abs(tot - ref_norm) < 1e-3 * max(1.0, ref_norm), (tot, ref_norm)
    after = float(torch.sqrt(sum((p.grad._t.float() ** 2).sum() for p in model.parameters())))
    assert after <= 1.05e-3, after                     # clipping did trigger on the true gradient scale
    before = model.fc1.weight._t.clone()
    scaler.step(opt)
    scaler.update()
    assert not torch.equal(model.fc1.weight._t, before)


def scenario_ddp_wire(a):
    """16-bit gradients on the wire (`gradient_dtype`): weight-gradient GEMMs write bf16 / fp16 into the buckets, the
    all-reduce accumulates in float32 and returns float32 gradients that match the float32-wire result to 16-bit
    rounding; overflow on one rank still skips the step on all ranks; a tied embedding adds its rows into the
    16-bit slot; the step replays from a CUDA graph."""
    from genesis_b200.models.transformers import TransformerConfig, QwenForCausalLM
    r, w, d = dist.get_rank(), dist.get_world_size(), dev(a.backend)
    cfg = TransformerConfig(vocab_size=512, hidden_size=128, intermediate_size=256, num_hidden_layers=2,
                            num_attention_heads=2, num_key_value_heads=1, head_dim=64, max_position_embeddings=128,
                            tie_word_embeddings=True)
    rs = np.random.RandomState(100 + r)
    tokens = torch.from_numpy(rs.randint(0, 512, (4, 65))).to(d)

    def grads(gradient_dtype, amp_dtype, scaler=None):
        genesis.manual_seed(11)
        m = QwenForCausalLM(cfg).to(d)
        net = nn.DistributedDataParallel(m, bucket_cap_mb=0.25, gradient_dtype=gradient_dtype, grad_scaler=scaler)
        idx = genesis.Tensor(tokens[:, :-1].contiguous())
        lab = genesis.Tensor(tokens[:, 1:].reshape(-1).contiguous())
        with genesis.amp.autocast(dtype=amp_dtype):
            loss = net(idx, labels=lab, return_logits=False)
        (scaler.scale(loss) if scaler is not None else loss).backward()
        torch.cuda.synchronize()
        dist.symm.check_status("ddp wire")
        return m, net, [p.grad._t.clone() for p in m.parameters()]

    _, net32, g32 = grads(None, genesis.bfloat16)
    mw, netw, gw = grads("bfloat16", genesis.bfloat16)
    assert any(b.wire is not None for b in netw._buckets) and not any(b.wire is not None for b in net32._buckets)
    for (name, p), a32, aw in zip(mw.named_parameters(), g32, gw):
        assert aw.dtype == torch.float32 and p.grad._t.data_ptr() == p._grad_buf.data_ptr(), name
        scale = max(float(a32.abs().max()), 1e-6)
        assert float((a32 - aw).abs().max()) <= 2e-2 * scale + 1e-6, (name, float((a32 - aw).abs().max()), scale)
    # every rank holds the same result
    for gth in gw[:3]:
        chk = gth.clone()
        tdist.broadcast(chk, 0)
        assert torch.equal(chk, gth)
    # fp16 wire with a GradScaler: values travel scaled, leave the kernel unscaled; an overflow reaches all ranks
    sc = genesis.amp.GradScaler(init_scale=256.0)
    m16, net16, g16 = grads("float16", genesis.float16, sc)
    for (name, p), a32, a16 in zip(m16.named_parameters(), g32, g16):
        scale = max(float(a32.abs().max()), 1e-6)
        assert float((a32 - a16).abs().max()) <= 3e-2 * scale + 1e-6, (name, float((a32 - a16).abs().max()), scale)
    assert not sc.found_inf()
    opt = genesis.optim.AdamW(m16.parameters(), lr=1e-3)
    sc.step(opt)
    sc.update()
    before = m16.model.layers[0].mlp.down_proj.weight._t.clone()
    opt.zero_grad()
    idx = genesis.Tensor(tokens[:, :-1].contiguous())
    lab = genesis.Tensor(tokens[:, 1:].reshape(-1).contiguous())
    with genesis.amp.autocast(dtype=genesis.float16):
        loss = net16(idx, labels=lab, return_logits=False)
    if r == w - 1:
        loss = loss * float("inf")
    sc.scale(loss).backward()
    sc.step(opt)
    assert sc.found_inf(), "overflow flag did not reach this rank"
    sc.update()
    assert torch.equal(m16.model.layers[0].mlp.down_proj.weight._t, before), "step was not skipped"
    # local accumulation under no_sync() stays in float32; the next synchronised step reduces the sum
    genesis.manual_seed(11)
    ma = QwenForCausalLM(cfg).to(d)
    neta = nn.DistributedDataParallel(ma, bucket_cap_mb=0.25, gradient_dtype="bfloat16")
    idx = genesis.Tensor(tokens[:, :-1].contiguous())
    lab = genesis.Tensor(tokens[:, 1:].reshape(-1).contiguous())
    with neta.no_sync(), genesis.amp.autocast(dtype=genesis.bfloat16):
        neta(idx, labels=lab, return_logits=False).backward()
    with genesis.amp.autocast(dtype=genesis.bfloat16):
        neta(idx, labels=lab, return_logits=False).backward()
    torch.cuda.synchronize()
    for (name, p), a32 in zip(ma.named_parameters(), g32):
        scale = max(float(a32.abs().max()), 1e-6)
        assert float((2 * a32 - p.grad._t).abs().max()) <= 5e-2 * scale + 1e-6, name
    # whole step from a CUDA graph, eager twin alongside
    def make():
        genesis.manual_seed(9)
        m = QwenForCausalLM(cfg).to(d)
        net = nn.DistributedDataParallel(m, bucket_cap_mb=0.25, gradient_dtype="bfloat16")
        o = genesis.optim.AdamW(m.parameters(), lr=1e-3)

        def step(tok):
            i_ = genesis.Tensor(tok._t[:, :-1].contiguous())
            l_ = genesis.Tensor(tok._t[:, 1:].reshape(-1).contiguous())
            with genesis.amp.autocast(dtype=genesis.bfloat16):
                ls = net(i_, labels=l_, return_logits=False)
            o.zero_grad()
            ls.backward()
            o.step()
            return ls
        return m, o, step
    ma, oa, step_a = make()
    mb, ob, step_b = make()
    batches = [genesis.Tensor(torch.from_numpy(rs.randint(0, 512, (4, 65))).to(d)) for _ in range(5)]
    graphed = genesis.cuda.GraphedTrainStep(step_b, ob, [batches[0]], warmup=2)
    for _ in range(2):
        step_a(batches[0])
    for i, t in enumerate(batches[1:]):
        la, lb = step_a(t), graphed(t)
        torch.cuda.synchronize()
        assert abs(float(la._t) - float(lb._t)) < 3e-3 * max(1.0, abs(float(la._t))), (i, float(la._t), float(lb._t))
    dist.symm.check_status("graphed ddp wire")


def scenario_ep(a):
    """Expert-parallel MoE layer equals the single-process layer holding all experts."""
    from genesis_b200.models.transformers.moe import MoELayer
    from genesis_b200.parallel.ep import EPGroup, mark_expert_parameters
    r, w, d = dist.get_rank(), dist.get_world_size(), dev(a.backend)
    H, E, k, I, T = 32, 4 * w, 2, 48, 24
    torch.manual_seed(5)
    genesis.manual_seed(5)
    full = MoELayer(H, E, k, I).to(d)                       # identical on every rank (same seed)
    ep_layer = MoELayer(H, E, k, I, ep_group=EPGroup()).to(d)
    ep_layer.gate.weight._t.copy_(full.gate.weight._t)
    lo = r * (E // w)
    for name in ("w_gate_up", "w_down"):
        getattr(ep_layer.experts, name)._t.copy_(getattr(full.experts, name)._t[lo:lo + E // w])
    assert mark_expert_parameters(ep_layer) == 2
    rs = np.random.RandomState(50 + r)
    xs = torch.from_numpy(rs.randn(w, 2, T // 2, H).astype(np.float32)).to(d)   # each rank builds only its own slice
    x_mine = torch.from_numpy(np.random.RandomState(50 + r).randn(2, T // 2, H).astype(np.float32)).to(d)
    xg, xe = genesis.Tensor(x_mine.clone(), requires_grad=True), genesis.Tensor(x_mine.clone(), requires_grad=True)
    full.train()
    ep_layer.train()
    of = full(xg)
    oe = ep_layer(xe)
    assert torch.allclose(of._t, oe._t, atol=1e-5, rtol=1e-4), float((of._t - oe._t).abs().max())
    gout = torch.from_numpy(np.random.RandomState(90 + r).randn(*of.shape).astype(np.float32)).to(d)
    (of * genesis.Tensor(gout)).sum().backward()
    (oe * genesis.Tensor(gout)).sum().backward()
    assert torch.allclose(xg.grad._t, xe.grad._t, atol=1e-5, rtol=1e-4)
    assert torch.allclose(full.gate.weight.grad._t, ep_layer.gate.weight.grad._t, atol=1e-5, rtol=1e-4)
    # expert gradients: the shard's gradient is the SUM over ranks of the full model's local gradients
    for name in ("w_gate_up", "w_down"):
        gfull = getattr(full.experts, name).grad._t.clone()
        tdist.all_reduce(gfull)
        got = getattr(ep_layer.experts, name).grad._t
        assert torch.allclose(got, gfull[lo:lo + E // w], atol=2e-5, rtol=1e-4), name
    del xs
    from genesis_b200.parallel import ep as ep_mod
    if a.backend == "nccl" and os.environ.get("GENESIS_COMM", "p2p") == "p2p":
        assert ep_mod.p2p_layers_run >= 1, "the peer-memory transport was not used"
        # bf16 under autocast at a size where every CTA has work: p2p transport against the NCCL transport
        H, E, k, I, T = 256, 8 * w, 4, 512, 4096
        genesis.manual_seed(7)
        layer = MoELayer(H, E, k, I, ep_group=EPGroup()).to(d)
        x0 = torch.from_numpy(np.random.RandomState(7 + r).randn(1, T, H).astype(np.float32)).to(d)
        outs, grads = [], []
        for mode in ("p2p", "nccl"):
            os.environ["GENESIS_COMM"] = mode
            xin = genesis.Tensor(x0.clone(), requires_grad=True)
            for p_ in layer.parameters():
                p_.grad = None
            with genesis.amp.autocast(dtype=genesis.bfloat16):
                o = layer(xin)
            (o.float() * o.float()).sum().backward()
            outs.append(o._t.float().clone())
            grads.append((xin.grad._t.float().clone(), layer.experts.w_down.grad._t.float().clone(),
                          layer.gate.weight.grad._t.float().clone()))
        os.environ["GENESIS_COMM"] = "p2p"
        assert torch.allclose(outs[0], outs[1], atol=2e-2, rtol=2e-2), float((outs[0] - outs[1]).abs().max())
        for g0, g1 in zip(grads[0], grads[1]):
            assert torch.allclose(g0, g1, atol=3e-2, rtol=3e-2), float((g0 - g1).abs().max())


def scenario_skipped_collective(a):
    """One rank does not enter a collective: the others get `CommTimeout` within the process-group budget instead of
    hanging (host-made failure, CPU ranks only; `GENESIS_COMM_TIMEOUT_S` is short in this scenario)."""
    import time
    from genesis_b200.distributed.process_group import CommTimeout
    r, w, d = dist.get_rank(), dist.get_world_size(), dev(a.backend)
    t = genesis.Tensor(torch.ones(8, device=d))
    dist.all_reduce(t)                                  # everyone takes part: fine
    assert float(t._t[0]) == w
    if r == w - 1:
        time.sleep(6.0)                                 # this rank "forgets" the next collective
    else:
        t0 = time.time()
        try:
            dist.all_reduce(t)
            raise AssertionError("all_reduce returned although a rank never joined")
        except CommTimeout:
            assert time.time() - t0 < 5.5
    # no further collective: the group is left as is and every process exits on its own


def scenario_heartbeat(a):
    """A rank that stops beating is reported by the others within the budget; nobody touches a GPU."""
    import time
    from genesis_b200.distributed.process_group import CommTimeout
    r, w = dist.get_rank(), dist.get_world_size()
    store = tdist.TCPStore("127.0.0.1", int(os.environ["MASTER_PORT"]) + 7, w, r == 0, wait_for_workers=True)
    hb = dist.Heartbeat(store, r, w, interval=0.05, timeout=0.6).start()
    time.sleep(0.5)
    hb.check()                                   # everyone alive
    if r == w - 1:
        hb.pause()                               # this rank "hangs" (stops beating) but keeps its process
        time.sleep(2.0)
    else:
        t0 = time.time()
        dead = []
        while time.time() - t0 < 3.0 and not dead:
            dead = hb.dead_ranks()
            time.sleep(0.05)
        assert dead == [w - 1], dead
        try:
            hb.check()
            raise AssertionError("check() did not raise")
        except CommTimeout as e:
            assert str(w - 1) in str(e)
        time.sleep(0.5)
    hb.stop()


SCENARIOS = {k[len("scenario_"):]: v for k, v in list(globals().items()) if k.startswith("scenario_")}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--scenario", required=True)
    ap.add_argument("--backend", default="gloo")
    a = ap.parse_args()
    if a.backend == "nccl":
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
    dist.init_process_group(backend=a.backend)
    try:
        SCENARIOS[a.scenario](a)
        if a.backend == "nccl":
            torch.cuda.synchronize()
        print(f"WORKER_OK {dist.get_rank()}", flush=True)
    finally:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
