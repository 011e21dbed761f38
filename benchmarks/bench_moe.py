"""Training-step benchmark of the Qwen3-MoE-shaped decoder with expert parallelism = data parallelism = world.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        benchmarks/bench_moe.py --steps 4 --warmup 3 [--layers L] [--transport p2p|nccl]

Model: 24 layers, hidden 2048, 32 query / 4 KV heads of 128, every layer MoE with 128 experts of SwiGLU width 768,
softmax router top-8 with renormalised weights, aux loss 0.001, vocab 151936; seq 4096, micro-batch 2 per GPU,
bf16 autocast, AdamW.  The full model holds 14.5 G expert parameters (232 GB of fp32 weights + Adam state), so it
needs the expert shards of 8 GPUs; `--layers` runs the same layer shape with fewer layers on fewer GPUs.
`--transport` picks how rows travel between ranks: the peer-memory pull kernels (default) or NCCL all-to-alls.
Prints one JSON line on rank 0; times with CUDA events, max over ranks.
"""
import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def parse(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--layers", type=int, default=24)
    ap.add_argument("--experts", type=int, default=128)
    ap.add_argument("--micro-batch", type=int, default=2)
    ap.add_argument("--seq-len", type=int, default=4096)
    ap.add_argument("--transport", default="p2p", choices=["p2p", "nccl"])
    ap.add_argument("--kernels", type=int, default=0, help="also list the N kernels with the most device time of one step")
    return ap.parse_args(argv)


def run(args, init_group=True):
    """One timed run; returns the result dict on rank 0 (None elsewhere).  `init_group=False`: the caller owns the
    process group (bench.py runs this after its dense model inside one job)."""
    os.environ["GENESIS_COMM"] = args.transport

    import numpy as np
    import torch
    import genesis_b200 as genesis
    from bench import ClockSampler, dist_env, time_steps
    from genesis_b200 import distributed as dist
    from genesis_b200.models.transformers import MoEForCausalLM, get_moe_config
    from genesis_b200.ops import native
    from genesis_b200.parallel.ep import EPGroup, mark_expert_parameters
    from genesis_b200.parallel import ep as ep_mod

    rank, world, local = dist_env(args)
    torch.cuda.set_device(local)
    if world > 1 and init_group:
        dist.init_process_group(backend="nccl")
    cfg = get_moe_config("qwen3-moe-bench")
    cfg.num_hidden_layers = args.layers
    cfg.num_local_experts = args.experts
    cfg.max_position_embeddings = args.seq_len
    genesis.manual_seed(1234)
    ep = EPGroup() if world > 1 else None
    model = MoEForCausalLM(cfg, ep_group=ep).cuda()
    if world > 1:
        mark_expert_parameters(model)
        net = genesis.nn.parallel.DistributedDataParallel(model, device_ids=[local], gradient_dtype="bfloat16")
    else:
        net = model
    opt = genesis.optim.AdamW(model.parameters(), lr=3e-4)
    # the optimizer kernel keeps the bf16 copies of the weights (and the K-major twins of the 2-D ones) current
    opt.enable_shadows(genesis.bfloat16, genesis.nn.utils.fused_parameter_groups(model))
    B, S = args.micro_batch, args.seq_len
    rs = np.random.RandomState(1000 + rank)
    host = [torch.from_numpy(rs.randint(0, cfg.vocab_size, (B, S)).astype(np.int64)).pin_memory() for _ in range(4)]
    counter = {"i": 0}

    def step():
        counter["i"] += 1
        tokens = host[counter["i"] % 4].to("cuda", non_blocking=True)
        idx = genesis.Tensor(tokens)
        with genesis.amp.autocast(dtype=genesis.bfloat16):
            loss = net(idx, labels=idx, return_logits=False)
        opt.zero_grad()
        loss.backward()
        opt.step()
        return loss

    sampler = ClockSampler(local)
    native.launch_count = 0
    if rank == 0:
        sampler.start()
    ms, last = time_steps(torch, step, args.steps, args.warmup, world)
    clocks = sampler.stop() if rank == 0 else None
    loss = float(last._t.float().cpu())
    kernels = None
    if args.kernels:
        from torch.profiler import profile, ProfilerActivity
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            step()
            torch.cuda.synchronize()
        rows = sorted(((e.device_time_total / 1e3, e.count, e.key[:90]) for e in prof.key_averages()
                       if e.device_time_total > 0), reverse=True)
        kernels = [{"ms": round(ms_, 3), "calls": n, "name": k} for ms_, n, k in rows[:args.kernels]]
    native.check_status()
    if world > 1:
        from genesis_b200.distributed import symm
        symm.check_status("moe step")
        if init_group:
            dist.destroy_process_group()
    comm = ep_mod.comm_profile() if world > 1 else None
    if rank != 0:
        return None
    n_params = sum(p._t.numel() for p in model.parameters())
    return {
        "metric": "MoE EP tokens/sec (box, max over ranks)", "value": B * S * world / (ms / 1e3), "unit": "tokens/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "dtype": "bf16", "data": "synthetic uniform token ids, random-init N(0,0.02) weights",
        "config": {"model": "qwen3-moe-bench", "layers": args.layers, "experts": args.experts, "top_k": 8,
                   "global_batch": B * world, "seq_len": S, "parallelism": f"ep{world} x dp{world}",
                   "transport": args.transport, "params_per_rank": n_params},
        "clocks": clocks, "loss": loss, "kernels": kernels, "comm": comm,
        "gpu_launches": native.launch_count // (args.steps + args.warmup) * args.steps,
    }


def main():
    out = run(parse())
    if out is not None:
        print(json.dumps(out), flush=True)


if __name__ == "__main__":
    main()
