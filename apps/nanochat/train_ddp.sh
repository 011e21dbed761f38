#!/bin/bash
# Data-parallel training on N GPUs of one node: ./train_ddp.sh N [extra train.py arguments]
# Reference counterpart: apps/nanochat/train_ddp.sh:21-31.
N=${1:-8}
shift
HERE="$(cd "$(dirname "$0")" && pwd)"
exec python -m torch.distributed.run --nnodes=1 --nproc-per-node "$N" --master-addr 127.0.0.1 --master-port "${MASTER_PORT:-29500}" \
    "$HERE/train.py" --ddp --batch-size 4 --block-size 2048 --amp --dtype bf16 "$@"
