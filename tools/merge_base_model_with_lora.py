"""Merge one or more LoRA adapters into a HuggingFace-format base model.

    python tools/merge_base_model_with_lora.py --base_model base_dir --lora_model a_dir[,b_dir] \
        --output_dir merged [--output_type huggingface]

Each adapter directory holds ``adapter_model.bin`` + ``adapter_config.json`` (peft schema — what
``tools/convert_ds_weight_to_hf_fast.py --lora_mode`` writes).  Adapters are folded in sequence:
``W += (alpha / r) · B · A``.  The merge is done natively on the state dicts (no peft needed).
"""
import argparse
import json
import os
import shutil
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from easyllm_b200.ckpt.hf_import import load_hf_state  # noqa: E402
from easyllm_b200.models.lora import merge_lora_into_hf_state  # noqa: E402


def main(argv=None):
    p = argparse.ArgumentParser()
    p.add_argument("--base_model", required=True)
    p.add_argument("--lora_model", required=True, help="comma separated adapter directories")
    p.add_argument("--output_dir", required=True)
    p.add_argument("--output_type", default="huggingface", choices=["huggingface", "pth"])
    p.add_argument("--tokenizer_path", default=None)
    a = p.parse_args(argv)
    state = load_hf_state(a.base_model)
    for d in a.lora_model.split(","):
        d = d.strip()
        with open(os.path.join(d, "adapter_config.json")) as f:
            cfg = json.load(f)
        adapter = torch.load(os.path.join(d, "adapter_model.bin"), map_location="cpu")
        # a tokenizer extended during fine-tuning: grow the embeddings to the adapter's vocabulary
        for key, tgt in (("base_model.model.model.embed_tokens.weight", "model.embed_tokens.weight"),
                         ("base_model.model.lm_head.weight", "lm_head.weight")):
            if key in adapter:
                state[tgt] = adapter.pop(key)
        state = merge_lora_into_hf_state(state, adapter, cfg["lora_alpha"] / cfg["r"])
        print(f"merged {d}")
    os.makedirs(a.output_dir, exist_ok=True)
    torch.save(state, os.path.join(a.output_dir, "pytorch_model.bin" if a.output_type == "huggingface" else "consolidated.pth"))
    for fn in os.listdir(a.base_model):
        if fn.endswith(".json") and "index" not in fn or fn.endswith(".model"):
            shutil.copy(os.path.join(a.base_model, fn), os.path.join(a.output_dir, fn))
    print(f"wrote {a.output_dir}")


if __name__ == "__main__":
    main()
