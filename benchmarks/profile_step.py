"""Where one training step spends its device time: every kernel of an eager step of a dense Qwen model, summed by name.

    python benchmarks/profile_step.py [--model qwen2.5-0.5b] [--micro-batch 8] [--seq-len 2048] [--weight-copies] [--top 40]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29511 \
        benchmarks/profile_step.py --weight-copies          (data-parallel step: rank 0 prints its kernels)

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
    ap.add_argument("--comm-timeline", action="store_true",
                    help="data-parallel runs: when each bucket all-reduce started and ended relative to the compute kernels")
    a = ap.parse_args()
    import torch
    from torch.profiler import profile, ProfilerActivity
    import genesis_b200 as genesis
    from genesis_b200.models.transformers import TransformerConfig, QwenForCausalLM
    from bench import CONFIGS

    cfg = TransformerConfig(**CONFIGS[a.model])
    genesis.manual_seed(0)
    world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    if world > 1:
        genesis.distributed.init_process_group(backend="nccl")
    model = QwenForCausalLM(cfg).cuda()
    net = genesis.nn.parallel.DistributedDataParallel(model, gradient_dtype=genesis.bfloat16) if world > 1 else model
    opt = genesis.optim.AdamW(model.parameters(), lr=3e-4)
    if a.weight_copies:
        opt.enable_shadows(genesis.bfloat16, genesis.nn.utils.fused_parameter_groups(model))
    tok = torch.randint(0, cfg.vocab_size, (a.micro_batch, a.seq_len + 1), device="cuda")

    def step():
        idx = genesis.Tensor(tok[:, :-1].contiguous())
        lab = genesis.Tensor(tok[:, 1:].reshape(-1).contiguous())
        with genesis.amp.autocast(dtype=genesis.bfloat16):
            loss = net(idx, labels=lab, return_logits=False)
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
    if rank == 0:
        print(f"host enqueue time {t_host * 1e3:.1f} ms, wall {t_all * 1e3:.1f} ms")
    with profile(activities=[ProfilerActivity.CUDA, ProfilerActivity.CPU]) as prof:
        step()
        torch.cuda.synchronize()
    if world > 1:
        genesis.distributed.barrier()
    if rank != 0:
        return
    if a.comm_timeline:
        evs = [e for e in prof.events() if e.device_type.name == "CUDA" and e.device_time_total > 0]
        t0 = min(e.time_range.start for e in evs)
        comm = [e for e in evs if "allreduce" in e.name]
        comp = [e for e in evs if "allreduce" not in e.name]
        end_comp = max(e.time_range.end for e in comp) - t0
        adam = [e for e in comp if "adam" in e.name]
        print(f"compute kernels end at {end_comp / 1e3:.2f} ms; optimizer kernel starts at "
              f"{(min(e.time_range.start for e in adam) - t0) / 1e3 if adam else -1:.2f} ms")
        for i, e in enumerate(sorted(comm, key=lambda e: e.time_range.start)):
            print(f"  all-reduce {i:3d}: start {(e.time_range.start - t0) / 1e3:8.2f} ms  duration {e.device_time_total / 1e3:7.3f} ms")
    rows = [(e.device_time_total / 1e3, e.count, e.key[:110]) for e in prof.key_averages()
            if e.device_time_total > 0 and e.device_type.name == "CUDA"]
    rows.sort(reverse=True)
    total = sum(r[0] for r in rows)
    print(f"total device ms {total:.2f} in {sum(r[1] for r in rows)} launches")
    for ms, n, name in rows[:a.top]:
        print(f"{ms:9.3f} ms {100 * ms / total:5.1f}%  x{n:5d}  {name}")


if __name__ == "__main__":
    main()
