#!/bin/bash
# Offline reference log-probs for DPO.  usage: sh scripts/mg_infer_logp.sh <num_gpus> <config.yaml> <out.jsonl>
ROOT=$(cd "$(dirname "$0")/.." && pwd)
export PYTHONPATH=$ROOT:$PYTHONPATH
python -m torch.distributed.run --nnodes=1 --nproc-per-node $1 --master-addr 127.0.0.1 --master-port ${PORT:-13335} \
  -m easyllm_b200.runners.base_llm_runner --config $2 --deepspeed --inference --generate-mode logp --logp-file $3 --launcher torch
