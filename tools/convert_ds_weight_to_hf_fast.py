"""Convert a layer-file (Megatron-DeepSpeed layout) checkpoint to a HuggingFace Llama
checkpoint, or a LoRA layer-file checkpoint to a peft adapter.

    python tools/convert_ds_weight_to_hf_fast.py --input_dir ckpt/global_step100 --output_dir out \
        --tp_size 2 --dim 4096 --n_heads 32 --num_key_value_heads 32 [--lora_mode]

Flags mirror the reference tool; dimensions left at their defaults are read from the tensors.
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from easyllm_b200.ckpt.ds_to_hf import convert, convert_lora  # noqa: E402


def main(argv=None):
    p = argparse.ArgumentParser()
    p.add_argument("--input_dir", required=True)
    p.add_argument("--output_dir", required=True)
    p.add_argument("--tp_size", type=int, default=None)
    p.add_argument("--dim", type=int, default=None)
    p.add_argument("--n_heads", type=int, default=None)
    p.add_argument("--n_layers", type=int, default=None, help="accepted for compatibility; derived from the files")
    p.add_argument("--intermediate_size", type=int, default=-1)
    p.add_argument("--num_key_value_heads", type=int, default=-1)
    p.add_argument("--norm_eps", type=float, default=1e-6)
    p.add_argument("--lora_mode", action="store_true")
    p.add_argument("--max_position_embeddings", type=int, default=2048)
    p.add_argument("--rope_theta", type=float, default=10000)
    a = p.parse_args(argv)
    if a.lora_mode:
        keys = convert_lora(a.input_dir, a.output_dir, a.tp_size)
        print(f"wrote adapter with {len(keys)} tensors to {a.output_dir}")
        return
    cfg = convert(a.input_dir, a.output_dir, a.tp_size, a.n_heads,
                  a.num_key_value_heads if a.num_key_value_heads > 0 else None, a.dim,
                  a.intermediate_size, a.norm_eps, a.max_position_embeddings, a.rope_theta)
    print(f"wrote HF checkpoint to {a.output_dir}: {cfg}")


if __name__ == "__main__":
    main()
