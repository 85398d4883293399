#!/bin/bash
# 3D-parallel inference.  usage: sh scripts/mg_infer.sh <num_gpus> <config.yaml> <mode: interactive|eval> [partition]
ROOT=$(cd "$(dirname "$0")/.." && pwd)
export PYTHONPATH=$ROOT:$PYTHONPATH
export NCCL_DEBUG=${NCCL_DEBUG:-WARN}
export TORCH_NCCL_ASYNC_ERROR_HANDLING=1   # a hung broadcast ends the job instead of blocking it
ARGS="--config $2 --deepspeed --inference --generate-mode ${3:-interactive} --top-k 40 --top-p 0.9 --temperature 0.2"
if [ -n "$4" ]; then
  srun -n$1 -p $4 --gres=gpu:$(($1 < 8 ? $1 : 8)) --ntasks-per-node=$(($1 < 8 ? $1 : 8)) \
    python -m easyllm_b200.runners.base_llm_runner $ARGS --launcher slurm
else
  python -m torch.distributed.run --nnodes=1 --nproc-per-node $1 --master-addr 127.0.0.1 --master-port ${PORT:-13334} \
    -m easyllm_b200.runners.base_llm_runner $ARGS --launcher torch
fi
