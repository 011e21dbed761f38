"""nanochat-style language-model trainer on genesis_b200.

    python apps/nanochat/train.py --data synthetic --max-steps 20 --amp --dtype bf16
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 apps/nanochat/train.py --ddp \
        --data /path/to/shards --tokenizer tokenizer.json --batch-size 4 --block-size 2048 --amp --dtype bf16

Same command line as the reference trainer (`--ddp --batch-size --block-size --learning-rate --accumulation-steps
--eval-interval --save-interval --max-steps --seed --amp --dtype --profile --profile-steps`), plus the data /
tokenizer / model / resume options this build adds.  One process per GPU; DDP buckets are all-reduced by the fused
peer-memory kernel while backward still runs; gradient accumulation skips the all-reduce on all but the last
micro-step; checkpoints are `genesis.save_checkpoint` files that `--resume` continues from (model, optimizer,
scaler, step).  Reference counterpart: apps/nanochat/train.py:59-409.
"""
import argparse
import os
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

MODELS = {
    # the reference trainer's model: 28 layers, 1536 wide, 24 heads of 64, dense attention, theta 1e4
    "nanochat": dict(num_hidden_layers=28, num_attention_heads=24, num_key_value_heads=24, hidden_size=1536,
                     intermediate_size=8960, head_dim=64, norm_eps=1e-6, rope_theta=10000.0),
    "qwen2.5-0.5b": dict(num_hidden_layers=24, num_attention_heads=14, num_key_value_heads=2, hidden_size=896,
                         intermediate_size=4864, head_dim=64, norm_eps=1e-6, rope_theta=1e6, tie_word_embeddings=True),
    "tiny": dict(num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, hidden_size=128,
                 intermediate_size=256, head_dim=32, norm_eps=1e-6, rope_theta=1e4),
}


def parse_args(argv=None):
    ap = argparse.ArgumentParser(description="Train a nanochat model")
    ap.add_argument("--ddp", action="store_true", help="data-parallel training (torchrun environment)")
    ap.add_argument("--batch-size", type=int, default=1, help="micro-batch per GPU")
    ap.add_argument("--block-size", type=int, default=2048, help="sequence length")
    ap.add_argument("--learning-rate", type=float, default=3e-4)
    ap.add_argument("--accumulation-steps", type=int, default=1)
    ap.add_argument("--eval-interval", type=int, default=500)
    ap.add_argument("--save-interval", type=int, default=100)
    ap.add_argument("--max-steps", type=int, default=None)
    ap.add_argument("--seed", type=int, default=42)
    ap.add_argument("--amp", action="store_true", help="mixed precision")
    ap.add_argument("--dtype", default="fp16", choices=["fp16", "bf16"])
    ap.add_argument("--profile", action="store_true", help="chrome trace of the first steps (rank 0)")
    ap.add_argument("--profile-steps", type=int, default=5)
    # additions
    ap.add_argument("--data", default="synthetic", help="'synthetic' or a directory of parquet / txt / npy shards")
    ap.add_argument("--tokenizer", default="bytes", help="'bytes', a tokenizers JSON file or a sentencepiece model")
    ap.add_argument("--vocab-size", type=int, default=None, help="vocabulary of synthetic data (default 65536)")
    ap.add_argument("--model", default="nanochat", choices=sorted(MODELS))
    ap.add_argument("--device", default=None, help="default: cuda when available, else cpu")
    ap.add_argument("--warmup-steps", type=int, default=0, help="linear warm-up, then cosine decay to --max-steps")
    ap.add_argument("--clip-grad", type=float, default=0.0)
    ap.add_argument("--weight-copies", action="store_true",
                    help="with --amp on CUDA: let the optimizer keep the bf16 / fp16 copies of the weights current")
    ap.add_argument("--cuda-graph", action="store_true",
                    help="capture the whole step (forward, backward, clipping, optimizer) as a CUDA graph after three "
                         "eager steps and replay it; needs CUDA, --accumulation-steps 1 and, with --ddp, the "
                         "peer-memory transport")
    ap.add_argument("--eval-batches", type=int, default=20)
    ap.add_argument("--out", default=os.path.join(os.path.dirname(os.path.abspath(__file__)), "checkpoints", "model"))
    ap.add_argument("--resume", default=None, help="checkpoint file to continue from")
    ap.add_argument("--metrics", default=None, help="JSONL file for per-step metrics (rank 0)")
    ap.add_argument("--log-interval", type=int, default=10)
    return ap.parse_args(argv)


def setup_ddp(args, genesis, dist, torch):
    if args.ddp and "RANK" in os.environ and "WORLD_SIZE" in os.environ:
        rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
        local = int(os.environ.get("LOCAL_RANK", 0))
        on_gpu = torch.cuda.is_available() and (args.device is None or args.device.startswith("cuda"))
        if on_gpu:
            torch.cuda.set_device(local)          # before the process group, so nothing lands on GPU 0
        dist.init_process_group(backend="nccl" if on_gpu else "gloo")
        return True, rank, local, world
    return False, 0, 0, 1


def main(argv=None):
    args = parse_args(argv)
    import numpy as np
    import torch
    import genesis_b200 as genesis
    import genesis_b200.nn as nn
    import genesis_b200.nn.functional as F
    from genesis_b200 import distributed as dist
    from genesis_b200.models.transformers import TransformerConfig, QwenForCausalLM
    from genesis_b200.optim.lr_scheduler import get_cosine_schedule_with_warmup
    from genesis_b200.utils.metrics import JsonlLogger
    import data as D

    ddp, rank, local, world = setup_ddp(args, genesis, dist, torch)
    device = args.device or ("cuda" if torch.cuda.is_available() else "cpu")
    if device == "cuda" and ddp:
        device = f"cuda:{local}"
    np.random.seed(args.seed)
    genesis.manual_seed(args.seed)
    log = print if rank == 0 else (lambda *a, **k: None)

    # ---- data -----------------------------------------------------------------------------------
    B, T = args.batch_size, args.block_size
    if args.data == "synthetic":
        vocab = args.vocab_size or 65536
        train_it = D.synthetic_batches(vocab, B, T, seed=args.seed * 1000 + rank)
        val_it = D.synthetic_batches(vocab, B, T, seed=args.seed * 1000 + 500 + rank)
    else:
        tok = D.load_tokenizer(args.tokenizer)
        vocab = args.vocab_size or tok.vocab_size
        train_it = D.batches(D.token_stream(D.list_shards(args.data, "train"), tok, rank, world), B, T)
        val_it = D.batches(D.token_stream(D.list_shards(args.data, "val"), tok, rank, world), B, T)
    train_loader, val_loader = D.Prefetcher(train_it, device), D.Prefetcher(val_it, device)

    # ---- model ----------------------------------------------------------------------------------
    cfg = TransformerConfig(vocab_size=vocab, max_position_embeddings=T, **MODELS[args.model])
    model = QwenForCausalLM(cfg).to(genesis.device(device))
    net = nn.DistributedDataParallel(model, device_ids=[local]) if ddp else model
    if ddp:
        dist.barrier()
    opt = genesis.optim.AdamW(model.parameters(), lr=args.learning_rate)
    amp_dtype = genesis.float16 if args.dtype == "fp16" else genesis.bfloat16
    if args.weight_copies and args.amp and device.startswith("cuda"):
        # the optimizer kernel keeps the compute-dtype copies of the weights current: no per-step conversions
        opt.enable_shadows(amp_dtype, nn.utils.fused_parameter_groups(model))
    sched = None
    if args.max_steps and (args.warmup_steps or args.max_steps):
        sched = get_cosine_schedule_with_warmup(opt, args.warmup_steps, args.max_steps)
    scaler = genesis.amp.GradScaler() if (args.amp and args.dtype == "fp16") else None
    if scaler is not None and ddp:
        net.set_grad_scaler(scaler)
    step = 0
    if args.resume:
        ck = genesis.load(args.resume)          # the whole dict: load_checkpoint() returns only the two state dicts
        model.load_state_dict(ck["model_state_dict"])
        opt.load_state_dict(ck["optimizer_state_dict"])
        step = int(ck.get("step", 0))
        if scaler is not None and ck.get("scaler") is not None:
            scaler.load_state_dict(ck["scaler"])
        if sched is not None:
            for _ in range(step):
                sched.step()
        log(f"resumed from {args.resume} at step {step}")
    n_params = sum(p.numel() for p in model.parameters())
    log(f"model {args.model}: {n_params:,} parameters, vocab {vocab}; batch {B} x {T}, lr {args.learning_rate}, "
        f"amp {'off' if not args.amp else args.dtype}, world {world}, accumulation {args.accumulation_steps}")
    os.makedirs(args.out, exist_ok=True)
    metrics = JsonlLogger(args.metrics, rank=rank)

    def loss_of(x, y):
        idx, tgt = genesis.Tensor(x), genesis.Tensor(y.reshape(-1))
        if args.amp:
            with genesis.amp.autocast(dtype=amp_dtype):
                logits = net(idx)
                return F.cross_entropy(F.reshape(logits, (-1, logits.shape[-1])), tgt)
        logits = net(idx)
        return F.cross_entropy(F.reshape(logits, (-1, logits.shape[-1])), tgt)

    def evaluate():
        model.eval()
        total = 0.0
        with genesis.no_grad():
            for _ in range(args.eval_batches):
                x, y = next(val_loader)
                total += float(loss_of(x, y).item())
        model.train()
        mean = total / max(args.eval_batches, 1)
        if ddp:
            t = genesis.Tensor(torch.tensor([mean], device=device))
            dist.all_reduce(t)
            mean = float(t._t.item()) / world
        return mean

    def save(tag):
        if rank == 0:
            path = os.path.join(args.out, f"checkpoint_{tag}.pth")
            genesis.save_checkpoint(model.state_dict(), opt.state_dict(), path, step=step,
                                    scaler=None if scaler is None else scaler.state_dict())
            log(f"saved {path}")
        if ddp:
            # the other ranks wait here on the host while rank 0 writes: without this they would already sit inside
            # the next step's gradient all-reduce, spending its device-side wait budget on a file write
            dist.barrier()

    prof = None
    if args.profile and rank == 0:
        from torch.profiler import profile, ProfilerActivity
        acts = [ProfilerActivity.CPU] + ([ProfilerActivity.CUDA] if device.startswith("cuda") else [])
        prof = profile(activities=acts)
        prof.__enter__()

    def graph_step(x, y):
        """The whole step with no host read, as `GraphedTrainStep` captures it."""
        opt.zero_grad()
        loss = loss_of(x._t, y._t)
        (scaler.scale(loss) if scaler is not None else loss).backward()
        if args.clip_grad > 0:
            if scaler is not None:
                scaler.unscale_(opt)
            nn.utils.clip_grad_norm_(model.parameters(), args.clip_grad, sync=False)
        if scaler is not None:
            scaler.step(opt)
            scaler.update()
        else:
            opt.step()
        return loss

    graphed = None
    if args.cuda_graph:
        if not device.startswith("cuda") or args.accumulation_steps != 1 or (ddp and not getattr(net, "_use_symm", False)):
            raise SystemExit("--cuda-graph needs CUDA, --accumulation-steps 1 and (with --ddp) the peer-memory transport")

    model.train()
    t0, tokens_since, loss_since, micro = time.time(), 0, 0.0, 0
    log("starting training")
    while args.max_steps is None or step < args.max_steps:
        if args.cuda_graph:
            if graphed is None:
                warm = [[genesis.Tensor(b) for b in next(train_loader)] for _ in range(3)]
                graphed = genesis.cuda.GraphedTrainStep(graph_step, opt, warm[0], warmup=3, warmup_inputs=warm)
                done = 3
                step_loss = graphed.static_outputs
                log("training step captured as a CUDA graph "
                    f"({graphed.kernels_per_step} kernels per replay) after 3 eager steps")
            else:
                x, y = next(train_loader)
                step_loss = graphed(x, y)
                done = 1
            for _ in range(done):
                if sched is not None:
                    sched.step()
                step += 1
                micro += 1
            tokens_since += B * T * world * done
            if step % args.log_interval < done or step == args.max_steps:
                lv = float(step_loss.item())
                dt = time.time() - t0
                log(f"step {step}: loss {lv:.4f}, {tokens_since / dt:,.0f} tokens/s")
                metrics.log(step=step, loss=lv, tokens_per_s=tokens_since / dt, lr=opt.lr)
                t0, tokens_since = time.time(), 0
            if args.eval_interval and step % args.eval_interval < done:
                log(f"step {step}: validation loss {evaluate():.4f}")
            if args.save_interval and step % args.save_interval < done:
                save(step)
            continue
        opt.zero_grad()
        step_loss = 0.0
        for a in range(args.accumulation_steps):
            x, y = next(train_loader)
            last = a == args.accumulation_steps - 1
            ctx = net.no_sync() if (ddp and not last) else _Null()
            with ctx:
                loss = loss_of(x, y)
                scaled = loss * (1.0 / args.accumulation_steps)
                (scaler.scale(scaled) if scaler is not None else scaled).backward()
            step_loss = loss          # keep the tensor: read on the host only when it is logged
            micro += 1
        if args.clip_grad > 0:
            if scaler is not None:
                scaler.unscale_(opt)
            nn.utils.clip_grad_norm_(model.parameters(), args.clip_grad)
        if scaler is not None:
            scaler.step(opt)
            scaler.update()
        else:
            opt.step()
        if sched is not None:
            sched.step()
        step += 1
        tokens_since += B * T * args.accumulation_steps * world
        if step % args.log_interval == 0 or step == args.max_steps:
            lv = float(step_loss.item())
            dt = time.time() - t0
            log(f"step {step}: loss {lv:.4f}, {tokens_since / dt:,.0f} tokens/s"
                + (f", scale {scaler.get_scale():.0f}" if scaler is not None else ""))
            metrics.log(step=step, loss=lv, tokens_per_s=tokens_since / dt, lr=opt.param_groups[0]["lr"]
                        if hasattr(opt, "param_groups") else args.learning_rate)
            t0, tokens_since = time.time(), 0
        if prof is not None and step >= args.profile_steps:
            prof.__exit__(None, None, None)
            trace = os.path.join(args.out, "trace.json")
            prof.export_chrome_trace(trace)
            log(f"profiler trace written to {trace}")
            prof = None
        if args.eval_interval and step % args.eval_interval == 0:
            log(f"step {step}: validation loss {evaluate():.4f}")
        if args.save_interval and step % args.save_interval == 0:
            save(step)
    save("final")
    metrics.close()
    if ddp:
        dist.destroy_process_group()
    return step


class _Null:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False


if __name__ == "__main__":
    main()
