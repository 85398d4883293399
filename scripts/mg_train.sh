#!/bin/bash
# 3D-parallel training.  usage: sh scripts/mg_train.sh <num_gpus> <config.yaml> [partition]
# torchrun on one node (default) or slurm when a partition is given.
ROOT=$(cd "$(dirname "$0")/.." && pwd)
export PYTHONPATH=$ROOT:$PYTHONPATH
export NCCL_DEBUG=${NCCL_DEBUG:-WARN}
export TORCH_NCCL_ASYNC_ERROR_HANDLING=1
if [ -n "$3" ]; then
  srun -n$1 -p $3 --gres=gpu:$(($1 < 8 ? $1 : 8)) --ntasks-per-node=$(($1 < 8 ? $1 : 8)) --cpus-per-task=16 \
    python -m easyllm_b200.runners.base_llm_runner --config $2 --launcher slurm
else
  python -m torch.distributed.run --nnodes=1 --nproc-per-node $1 --master-addr 127.0.0.1 --master-port ${PORT:-13333} \
    --max-restarts 0 -m easyllm_b200.runners.base_llm_runner --config $2 --launcher torch
fi
