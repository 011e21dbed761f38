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
