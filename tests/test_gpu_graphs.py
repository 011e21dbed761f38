"""CUDA-graph capture of the framework's kernels: a captured forward (and forward + backward) replays to the same
numbers as eager execution, with one launch per replay."""
import pytest
import torch

import genesis_b200 as genesis
import genesis_b200.nn as nn
from genesis_b200.ops import native

pytestmark = pytest.mark.gpu


def test_captured_forward_matches_eager_and_launches_nothing_on_replay():
    genesis.manual_seed(0)
    model = nn.Sequential(nn.Linear(256, 512), nn.ReLU(), nn.RMSNorm(512), nn.Linear(512, 64)).cuda()
    x0 = genesis.randn(128, 256, device="cuda")

    def fwd(x):
        with genesis.no_grad(), genesis.amp.autocast(dtype=genesis.bfloat16):
            return model(x)

    graphed = genesis.cuda.make_graphed_callable(fwd, [x0])
    for seed in (1, 2, 3):
        x = genesis.Tensor(torch.randn(128, 256, device="cuda", generator=torch.Generator("cuda").manual_seed(seed)))
        ref = fwd(x)._t.float().clone()
        before = native.launch_count
        out = graphed(x)
        assert native.launch_count == before                     # nothing goes through the Python launch path
        torch.cuda.synchronize()
        assert torch.allclose(out._t.float(), ref, atol=1e-2, rtol=1e-2)


def test_captured_forward_backward_gives_eager_gradients():
    genesis.manual_seed(1)
    model = nn.Sequential(nn.Linear(64, 128), nn.SiLU(), nn.Linear(128, 8)).cuda()
    params = list(model.parameters())

    def step(x, y):
        for p in params:
            if p.grad is not None:
                p.grad._t.zero_()
        loss = ((model(x) - y) * (model(x) - y)).sum()
        loss.backward()
        return loss

    x = genesis.randn(32, 64, device="cuda")
    y = genesis.randn(32, 8, device="cuda")
    step(x, y)                                                   # creates the .grad tensors the graph will reuse
    graphed = genesis.cuda.make_graphed_callable(step, [x, y], warmup=2)
    x2, y2 = genesis.randn(32, 64, device="cuda"), genesis.randn(32, 8, device="cuda")
    graphed(x2, y2)
    torch.cuda.synchronize()
    got = [p.grad._t.clone() for p in params]
    step(x2, y2)
    torch.cuda.synchronize()
    for g, p in zip(got, params):
        assert torch.allclose(g, p.grad._t, atol=1e-4, rtol=1e-4)


def _tiny_lm(seed):
    from genesis_b200.models.transformers import TransformerConfig, QwenForCausalLM
    genesis.manual_seed(seed)
    cfg = TransformerConfig(vocab_size=512, hidden_size=128, intermediate_size=256, num_hidden_layers=2,
                            num_attention_heads=2, num_key_value_heads=1, head_dim=64, max_position_embeddings=128,
                            rope_theta=1e4, norm_eps=1e-6, attention_bias=True)
    return QwenForCausalLM(cfg).cuda()


def _lm_step(model, opt):
    def step(tokens):
        idx = genesis.Tensor(tokens._t[:, :-1].contiguous())
        labels = genesis.Tensor(tokens._t[:, 1:].reshape(-1).contiguous())
        with genesis.amp.autocast(dtype=genesis.bfloat16):
            loss = model(idx, labels=labels, return_logits=False)
        opt.zero_grad()
        loss.backward()
        opt.step()
        return loss
    return step


def test_capturable_adamw_matches_host_scalars():
    """Step count, bias corrections and learning rate read from the device vector give the same parameters as the
    by-value launch arguments, including after a learning-rate change (fixed gradients: the update is elementwise,
    so both runs are bit-for-bit repeatable)."""
    g = torch.Generator("cuda").manual_seed(0)
    shapes = [(257, 33), (4096,), (64, 128)]
    init = [torch.randn(s, device="cuda", generator=g) for s in shapes]
    pa = [genesis.Tensor(t.clone(), requires_grad=True) for t in init]
    pb = [genesis.Tensor(t.clone(), requires_grad=True) for t in init]
    oa = genesis.optim.AdamW(pa, lr=1e-3, weight_decay=0.1)
    ob = genesis.optim.AdamW(pb, lr=1e-3, weight_decay=0.1).make_capturable()
    for i in range(6):
        if i == 3:
            oa.lr = ob.lr = 3e-4
        for x, y in zip(pa, pb):
            gr = torch.randn(x.shape, device="cuda", generator=g)
            x.grad = genesis.Tensor(gr.clone())
            y.grad = genesis.Tensor(gr.clone())
        oa.step()
        ob.step()
    torch.cuda.synchronize()
    for x, y in zip(pa, pb):
        assert torch.allclose(x._t, y._t, atol=1e-7, rtol=1e-6)
    assert float(ob._dyn[3]) == 6.0 and ob.t == 6
    # a state dict written by one optimizer restores the device step count of the other
    ob.load_state_dict(oa.state_dict())
    assert float(ob._dyn[3]) == 6.0 and abs(float(ob._dyn[0]) - 3e-4) < 1e-9


def test_graphed_train_step_follows_the_eager_trajectory():
    """A whole step (forward, backward, AdamW) replayed from a graph tracks eager training on the same batches: same
    losses, one graph launch per step, learning-rate change honoured, and parameters as close to an eager run as
    a second eager run is (kernels that accumulate with atomics differ in the last bits between runs, and Adam turns
    the sign flip of a near-zero gradient into a full-size update of that element)."""
    a, b, c = _tiny_lm(5), _tiny_lm(5), _tiny_lm(5)
    oa, ob, oc = (genesis.optim.AdamW(m.parameters(), lr=1e-3) for m in (a, b, c))
    sa, sc = _lm_step(a, oa), _lm_step(c, oc)
    g = torch.Generator("cuda").manual_seed(1)
    batches = [genesis.Tensor(torch.randint(0, 512, (4, 65), device="cuda", generator=g)) for _ in range(7)]
    warm = batches[0]
    graphed = genesis.cuda.GraphedTrainStep(_lm_step(b, ob), ob, [warm], warmup=2)
    assert graphed.kernels_per_step > 20
    for _ in range(2):
        sa(warm)                                                 # the two warm-up steps were real steps on `warm`
        sc(warm)
    assert ob.t == 2 and oa.t == 2
    for i, t in enumerate(batches[1:]):
        if i == 3:
            oa.lr = ob.lr = oc.lr = 2e-4
        la = sa(t)
        sc(t)
        before = native.launch_count
        lb = graphed(t)
        assert native.launch_count == before
        torch.cuda.synchronize()
        assert abs(float(la._t) - float(lb._t)) < 2e-3 * max(1.0, abs(float(la._t)))
    assert ob.t == oa.t == 8

    def gap(m1, m2):
        return max(float((p._t - q._t).abs().mean()) for p, q in zip(m1.parameters(), m2.parameters()))
    assert gap(a, b) <= 3.0 * gap(a, c) + 2e-5, (gap(a, b), gap(a, c))
    native.check_status()


def test_clip_grad_norm_without_host_read_matches_torch():
    import genesis_b200.nn as gnn
    g = torch.Generator("cuda").manual_seed(4)
    shapes = [(300, 70), (1025,), (64, 64, 3)]
    for max_norm in (0.5, 1e6):
        params = []
        for s in shapes:
            p = genesis.Tensor(torch.zeros(s, device="cuda"), requires_grad=True)
            p.grad = genesis.Tensor(torch.randn(s, device="cuda", generator=g))
            params.append(p)
        ref = [p.grad._t.clone().requires_grad_(False) for p in params]
        leaves = [torch.zeros_like(r, requires_grad=True) for r in ref]
        for leaf, r in zip(leaves, ref):
            leaf.grad = r.clone()
        want = torch.nn.utils.clip_grad_norm_(leaves, max_norm)
        got = gnn.utils.clip_grad_norm_(params, max_norm, sync=False)
        assert isinstance(got, genesis.Tensor)
        assert torch.allclose(got._t, want, rtol=1e-5)
        for p, leaf in zip(params, leaves):
            assert torch.allclose(p.grad._t, leaf.grad, rtol=1e-5, atol=1e-7)
        # the reading form gives a float and the same gradients
        for p, r in zip(params, ref):
            p.grad = genesis.Tensor(r.clone())
        total = gnn.utils.clip_grad_norm_(params, max_norm)
        assert isinstance(total, float) and abs(total - float(want)) < 1e-4 * float(want)
        for p, leaf in zip(params, leaves):
            assert torch.allclose(p.grad._t, leaf.grad, rtol=1e-5, atol=1e-7)


def test_trainer_app_with_cuda_graph(tmp_path):
    """The training app with --cuda-graph: three eager steps, capture, replays; logs finite losses and saves."""
    import importlib
    import json
    import os
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, os.path.join(root, "apps", "nanochat"))
    train = importlib.import_module("train")
    metrics = str(tmp_path / "m.jsonl")
    n = train.main(["--model", "tiny", "--data", "synthetic", "--vocab-size", "512", "--batch-size", "4",
                    "--block-size", "64", "--device", "cuda", "--out", str(tmp_path / "ck"), "--max-steps", "9",
                    "--log-interval", "3", "--eval-interval", "0", "--save-interval", "0", "--amp", "--dtype", "bf16",
                    "--clip-grad", "1.0", "--warmup-steps", "2", "--cuda-graph", "--weight-copies",
                    "--metrics", metrics])
    assert n == 9
    rows = [json.loads(l) for l in open(metrics)]
    assert [r["step"] for r in rows] == [3, 6, 9]
    assert all(r["loss"] == r["loss"] and r["loss"] < 10 for r in rows)
    assert os.path.exists(str(tmp_path / "ck" / "checkpoint_final.pth"))


@pytest.mark.parametrize("lp", ["bfloat16", "float16"])
def test_adamw_kernel_writes_current_low_precision_copies(lp):
    """The optimizer kernel's 16-bit copies (vector path on aligned tensors, scalar path on an odd-sized one and on a
    misaligned slice) equal a conversion of the updated parameters, and the update itself is unchanged by them."""
    td = getattr(torch, lp)
    g = torch.Generator("cuda").manual_seed(2)
    shapes = [(300, 64), (8192 * 3 + 5,), (7, 3), (5, 3)]
    init = [torch.randn(s, device="cuda", generator=g) for s in shapes]
    pa = [genesis.Tensor(t.clone(), requires_grad=True) for t in init]
    pb = [genesis.Tensor(t.clone(), requires_grad=True) for t in init]
    oa = genesis.optim.AdamW(pa, lr=1e-2)
    ob = genesis.optim.AdamW(pb, lr=1e-2)
    ob.enable_shadows(getattr(genesis, lp), groups=[[pb[0]], [pb[2], pb[3]]])   # pb[3]'s slice starts 42 bytes in
    try:
        for _ in range(3):
            for x, y in zip(pa, pb):
                gr = torch.randn(x.shape, device="cuda", generator=g)
                x.grad, y.grad = genesis.Tensor(gr.clone()), genesis.Tensor(gr.clone())
            oa.step()
            ob.step()
        torch.cuda.synchronize()
        for i, (x, y) in enumerate(zip(pa, pb)):
            assert torch.equal(x._t, y._t)
            assert torch.equal(ob._shadows[i], y._t.to(td))
    finally:
        ob.disable_shadows()
    native.check_status()


def test_graphed_fp16_step_with_grad_scaler_and_weight_copies():
    """fp16 autocast + GradScaler + optimizer-kept fp16 weight copies inside one captured step: tracks the eager
    run, the loss scale grows on the device across replays, and an overflow step is skipped in both."""
    def build():
        m = _tiny_lm(7)
        o = genesis.optim.AdamW(m.parameters(), lr=1e-3)
        sc = genesis.amp.GradScaler(init_scale=2.0 ** 10, growth_interval=3)

        def step(tokens):
            idx = genesis.Tensor(tokens._t[:, :-1].contiguous())
            labels = genesis.Tensor(tokens._t[:, 1:].reshape(-1).contiguous())
            with genesis.amp.autocast(dtype=genesis.float16):
                loss = m(idx, labels=labels, return_logits=False)
            o.zero_grad()
            sc.scale(loss).backward()
            sc.step(o)
            sc.update()
            return loss
        return m, o, sc, step

    a, oa, sa_, step_a = build()
    b, ob, sb_, step_b = build()
    ob.enable_shadows(genesis.float16, genesis.nn.utils.fused_parameter_groups(b))
    try:
        g = torch.Generator("cuda").manual_seed(3)
        batches = [genesis.Tensor(torch.randint(0, 512, (4, 65), device="cuda", generator=g)) for _ in range(8)]
        graphed = genesis.cuda.GraphedTrainStep(step_b, ob, [batches[0]], warmup=2)
        for _ in range(2):
            step_a(batches[0])
        for t in batches[1:]:
            la, lb = step_a(t), graphed(t)
            torch.cuda.synchronize()
            assert abs(float(la._t) - float(lb._t)) < 2e-3 * max(1.0, abs(float(la._t)))
        assert sa_.get_scale() == sb_.get_scale() and sb_.get_scale() > 2.0 ** 10      # grew inside the replays
        # the two models take different kernel paths (K-major weight twins and the fused MLP backward in `b`), so
        # they differ in rounding; Adam turns a sign flip of a near-zero gradient into a full learning-rate step
        gap = max(float((p._t - q._t).abs().mean()) for p, q in zip(a.parameters(), b.parameters()))
        assert gap < 5e-4, gap
    finally:
        ob.disable_shadows()
    native.check_status()
