"""CPU correctness run: MLP Linear(784->256) -> ReLU -> Dropout(0.2) -> Linear(256->10), batch 64, fp32, seed 0,
AdamW (lr 1e-3, wd 0.01), CrossEntropyLoss, 100 steps; then a genesis.save / genesis.load round trip.
Prints one JSON line with the loss curve ends, the round-trip check and the time per step.
"""
import json
import os
import sys
import tempfile
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    import numpy as np
    import genesis_b200 as genesis
    import genesis_b200.nn as nn
    genesis.manual_seed(0)
    rs = np.random.RandomState(0)
    model = nn.Sequential(nn.Linear(784, 256), nn.ReLU(), nn.Dropout(0.2), nn.Linear(256, 10))
    opt = genesis.optim.AdamW(model.parameters(), lr=1e-3, weight_decay=0.01)
    crit = nn.CrossEntropyLoss()
    x = genesis.tensor(rs.randn(64, 784).astype(np.float32))
    y = genesis.tensor(rs.randint(0, 10, size=64).astype(np.int64))
    losses = []
    t0 = time.perf_counter()
    for _ in range(100):
        opt.zero_grad()
        loss = crit(model(x), y)
        loss.backward()
        opt.step()
        losses.append(float(loss.item()))
    dt = (time.perf_counter() - t0) / 100
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "mlp.pth")
        genesis.save(model.state_dict(), path)
        sd = genesis.load(path)
    same = all(np.array_equal(sd[k].numpy(), v.numpy()) for k, v in model.state_dict().items())
    print(json.dumps({"config": "mlp 784-256-10, batch 64, fp32, cpu", "first_loss": losses[0], "last_loss": losses[-1],
                      "save_load_round_trip": same, "ms_per_step": dt * 1e3}))


if __name__ == "__main__":
    main()
