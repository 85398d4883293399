#!/bin/bash
# usage: sh scripts/convert_ds_weight_to_hf.sh <ckpt_dir/global_stepN> <out_dir> <tp_size> [extra converter flags]
ROOT=$(cd "$(dirname "$0")/.." && pwd)
export LOADWORKER=${LOADWORKER:-8}
python $ROOT/tools/convert_ds_weight_to_hf_fast.py --input_dir $1 --output_dir $2 --tp_size $3 "${@:4}"
