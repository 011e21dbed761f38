#!/bin/bash
# Single-GPU launch of the nanochat trainer (the multi-GPU form is train_ddp.sh).
#   ./train.sh [extra train.py arguments]
cd "$(dirname "$0")"
export CUDA_VISIBLE_DEVICES=${CUDA_VISIBLE_DEVICES:-0}
python train.py --data synthetic --amp --dtype bf16 --max-steps 1000 "$@"
