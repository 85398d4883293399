"""Offline build of the ``.bin/.idx`` token cache (and index maps) of a ``mmap_index_json`` dataset
from a training YAML, so the first training job does not pay for it (tools/build_index_mmap.py:18-58).

    python tools/build_index_mmap.py --config configs/megatron/mmap_llama_7b_sft.yaml [--splits 1]
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main(argv=None):
    from easyllm_b200.config import load_yaml
    from easyllm_b200.data import build_dataset, build_tokenizer
    p = argparse.ArgumentParser()
    p.add_argument("--config", required=True)
    p.add_argument("--data_type", default="train")
    p.add_argument("--splits", type=int, default=None)
    a = p.parse_args(argv)
    cfg = load_yaml(a.config)
    tok = build_tokenizer(cfg["tokenizer"])
    ds_cfg = cfg["data"][a.data_type]["dataset"]
    if ds_cfg["type"] != "mmap_index_json":
        raise SystemExit("the dataset of this config is not mmap_index_json")
    if a.splits:
        ds_cfg.setdefault("kwargs", {})["cache_splits"] = a.splits
    ds = build_dataset(ds_cfg, tok)
    print(f"built cache with {len(ds)} samples under {ds.cache_prefix}")


if __name__ == "__main__":
    main()
