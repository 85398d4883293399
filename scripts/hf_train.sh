#!/bin/bash
# HF-style data-parallel training.  usage: sh scripts/hf_train.sh <num_gpus> <config.yaml> [partition]
ROOT=$(cd "$(dirname "$0")/.." && pwd)
export PYTHONPATH=$ROOT:$PYTHONPATH
if [ -n "$3" ]; then
  srun -n$1 -p $3 --gres=gpu:$(($1 < 8 ? $1 : 8)) --ntasks-per-node=$(($1 < 8 ? $1 : 8)) \
    python -m easyllm_b200.runners.hf_runner --config $2 --launcher slurm
else
  python -m torch.distributed.run --nnodes=1 --nproc-per-node $1 --master-addr 127.0.0.1 --master-port ${PORT:-13336} \
    -m easyllm_b200.runners.hf_runner --config $2 --launcher torch
fi
