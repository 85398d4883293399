#!/bin/bash
# HF-style inference.  usage: sh scripts/hf_infer.sh <num_gpus> <config.yaml> [interactive|eval]
ROOT=$(cd "$(dirname "$0")/.." && pwd)
export PYTHONPATH=$ROOT:$PYTHONPATH
python -m torch.distributed.run --nnodes=1 --nproc-per-node $1 --master-addr 127.0.0.1 --master-port ${PORT:-13337} \
  -m easyllm_b200.runners.hf_runner --config $2 --inference --generate-mode ${3:-interactive} --launcher torch
