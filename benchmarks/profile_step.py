"""Where one training step spends its device time: every kernel of an eager step of a dense Qwen model, summed by name.

    python benchmarks/profile_step.py [--model qwen2.5-0.5b] [--micro-batch 8] [--seq-len 2048] [--weight-copies] [--top 40]

Runs three warm-up steps, measures how long the host needs to enqueue one step against its wall time (is the loop
launch-bound?), then records one step with torch.profiler's CUDA activity and prints the kernels by total time.
Profiler timings are for SHARES; the step time itself comes from `bench.py` (CUDA events, no profiler attached).
`--weight-copies` lets the optimizer keep the bf16 copies of the weights current, as `bench.py` does by default.
"""
import argparse
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="qwen2.5-0.5b")
    ap.add_argument("--micro-batch", type=int, default=8)
    ap.add_argument("--seq-len", type=int, default=2048)
    ap.add_argument("--weight-copies", action="store_true")
    ap.add_argument("--top", type=int, default=40)
    a = ap.parse_args()
    import torch
    from torch.profiler import profile, ProfilerActivity
    import genesis_b200 as genesis
    from genesis_b200.models.transformers import TransformerConfig, QwenForCausalLM
    from bench import CONFIGS

    cfg = TransformerConfig(**CONFIGS[a.model])
    genesis.manual_seed(0)
    model = QwenForCausalLM(cfg).cuda()
    opt = genesis.optim.AdamW(model.parameters(), lr=3e-4)
    if a.weight_copies:
        opt.enable_shadows(genesis.bfloat16, genesis.nn.utils.fused_parameter_groups(model))
    tok = torch.randint(0, cfg.vocab_size, (a.micro_batch, a.seq_len + 1), device="cuda")

    def step():
        idx = genesis.Tensor(tok[:, :-1].contiguous())
        lab = genesis.Tensor(tok[:, 1:].reshape(-1).contiguous())
        with genesis.amp.autocast(dtype=genesis.bfloat16):
            loss = model(idx, labels=lab, return_logits=False)
        opt.zero_grad()
        loss.backward()
        opt.step()
        return loss

    for _ in range(3):
        step()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    step()
    t_host = time.perf_counter() - t0
    torch.cuda.synchronize()
    t_all = time.perf_counter() - t0
    print(f"host enqueue time {t_host * 1e3:.1f} ms, wall {t_all * 1e3:.1f} ms")
    with profile(activities=[ProfilerActivity.CUDA, ProfilerActivity.CPU]) as prof:
        step()
        torch.cuda.synchronize()
    rows = [(e.device_time_total / 1e3, e.count, e.key[:110]) for e in prof.key_averages()
            if e.device_time_total > 0 and e.device_type.name == "CUDA"]
    rows.sort(reverse=True)
    total = sum(r[0] for r in rows)
    print(f"total device ms {total:.2f} in {sum(r[1] for r in rows)} launches")
    for ms, n, name in rows[:a.top]:
        print(f"{ms:9.3f} ms {100 * ms / total:5.1f}%  x{n:5d}  {name}")


if __name__ == "__main__":
    main()
