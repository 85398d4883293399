#!/bin/bash
# usage: sh scripts/convert_bin.sh <tokenizer_path> <data.jsonl> <out_dir> [bin_size]
ROOT=$(cd "$(dirname "$0")/.." && pwd)
python $ROOT/tools/build_pretrain_bin.py --tokenizer_path $1 --jsonl $2 --out_dir $3 --bin_size ${4:-262144}
