#!/bin/bash
# Runs the single-GPU benchmark drivers one after the other and keeps their JSON lines under ./bench_out/.
#   benchmarks/run.sh [quick]
cd "$(dirname "$0")/.."
out=bench_out
mkdir -p "$out"
q=""
[ "$1" = "quick" ] && q="--quick"
python bench.py --gpus 1                                            | tee "$out/train_qwen05b.json"
python bench.py --impl torch                                        | tee "$out/train_qwen05b_torch.json"
python benchmarks/bench_kernels.py --torch --what gemm,attn,adamw $q | tee "$out/kernels_gemm_attn.jsonl"
python benchmarks/bench_kernels.py --what norm,softmax,addnorm       | tee "$out/kernels_rows.jsonl"
python benchmarks/bench_ops.py --report "$out/ops.md"
python benchmarks/bench_pool.py                                     | tee "$out/pool.jsonl"
python benchmarks/profile_step.py --weight-copies                   | tee "$out/step_profile.txt"
