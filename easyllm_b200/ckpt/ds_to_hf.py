"""Layer-file checkpoint (TP-sharded) → HuggingFace Llama checkpoint.

Parity: tools/convert_ds_weight_to_hf_fast.py:205-531.  Layer ids are positions in the model's
spec list: ``1`` embedding, ``3 … n+2`` decoder blocks (HF layer ``id − 3``), ``n+4`` final
norm, ``n+5`` LM head, hence ``n_layers = max_id − 5``.  TP shards are merged by a rule per
tensor name: column-parallel → concatenate rows, row-parallel → concatenate columns,
replicated (norms, row-parallel bias) → average, packed ``wqkv`` → split every shard into its
q / k / v parts by GQA group, then concatenate.  Output: one ``pytorch_model-000NN-of-000MM.bin``
per block (+ one for embedding/norm/head), ``pytorch_model.bin.index.json`` and a
``LlamaConfig``.  LoRA mode writes a peft ``adapter_model.bin`` + ``adapter_config.json``.

Unlike the reference tool, model dimensions are read from the tensors themselves (flags only
override), and q/k/v biases (Qwen-style) are carried through.
"""
from __future__ import annotations

import glob
import json
import os
import re
import shutil
from concurrent.futures import ThreadPoolExecutor

import torch

from .layer_files import LAYER_RE, safe_load

COL = re.compile(r"(mlp\.(gate|up)_proj|self_attn\.(q|k|v)_proj)\.(weight|bias)$|word_embeddings\.weight$")
ROW = re.compile(r"(mlp\.down_proj|self_attn\.o_proj)\.weight$")
PACK = re.compile(r"self_attn\.wqkv\.(weight|bias)$")
MEAN = re.compile(r"(layernorm\.weight|^weight|^bias|rotary_emb\.inv_freq|o_proj\.bias|down_proj\.bias)$")
LORA_COL = re.compile(r"((gate|up|q|k|v)_proj\.lora_B_weight|word_embeddings\.lora_embedding_A_weight)$")
LORA_ROW = re.compile(r"(down|o)_proj\.lora_A_weight$")
LORA_MEAN = re.compile(r"((gate|up|q|k|v)_proj\.lora_A_weight|(down|o)_proj\.lora_B_weight|"
                       r"word_embeddings\.lora_embedding_B_weight)$")


def index_layer_files(load_dir):
    """{layer id: {tp rank: path}} and the decoder depth ``max_id − 5``."""
    table = {}
    for p in glob.glob(os.path.join(load_dir, "layer_*-model_*-model_states.pt")):
        m = LAYER_RE.search(os.path.basename(p))
        if m:
            table.setdefault(int(m.group(1)), {})[int(m.group(2))] = p
    if not table:
        raise FileNotFoundError(f"no layer_XX-model_YY-model_states.pt files under {load_dir}")
    return table, max(table) - 5


def _read_shards(files, tp_size, lid):
    if tp_size != len(files):
        raise ValueError(f"layer {lid}: found {len(files)} TP shards, expected {tp_size}")
    out = []
    for r in range(tp_size):
        if r not in files:
            raise ValueError(f"Pt file of layer {lid}, tp_rank {r} is not found")
        out.append(safe_load(files[r]))
    return out


def merge_tensor(name, shards, n_heads=None, n_kv_heads=None):
    """Merge the TP shards of one tensor; returns {hf suffix: tensor}."""
    tp = len(shards)
    if PACK.search(name):
        gs = n_heads // n_kv_heads
        unit = shards[0].shape[0] // (gs + 2)
        q = torch.cat([s[:unit * gs] for s in shards], 0)
        k = torch.cat([s[unit * gs:unit * (gs + 1)] for s in shards], 0)
        v = torch.cat([s[unit * (gs + 1):] for s in shards], 0)
        return {name.replace("wqkv", "q_proj"): q, name.replace("wqkv", "k_proj"): k, name.replace("wqkv", "v_proj"): v}
    if COL.search(name) or LORA_COL.search(name):
        return {name: torch.cat(shards, 0)}
    if ROW.search(name) or LORA_ROW.search(name):
        return {name: torch.cat(shards, 1)}
    if MEAN.search(name) or LORA_MEAN.search(name):
        return {name: (sum(s.float() for s in shards) / tp).to(shards[0].dtype)}
    raise KeyError(f"Not recognized key {name}")


def convert(input_dir, output_dir, tp_size=None, n_heads=None, num_key_value_heads=None, dim=None,
            intermediate_size=None, norm_eps=1e-6, max_position_embeddings=2048, rope_theta=10000.0,
            workers=None, dtype=None):
    """Write an HF Llama checkpoint; returns the LlamaConfig kwargs used."""
    if os.path.abspath(output_dir) == os.path.abspath(input_dir):
        output_dir = os.path.join(output_dir, "convert_hf")
    os.makedirs(output_dir, exist_ok=True)
    table, n_layer = index_layer_files(input_dir)
    tp_size = tp_size or len(table[1])
    total = n_layer + 1
    index = {"weight_map": {}}
    counts = []

    def emit(state, shard_no):
        fn = f"pytorch_model-{shard_no:05d}-of-{total:05d}.bin"
        if dtype is not None:
            state = {k: v.to(dtype) for k, v in state.items()}
        torch.save(state, os.path.join(output_dir, fn))
        for k, v in state.items():
            index["weight_map"][k] = fn
            counts.append(v.numel())

    special = {}
    for lid, hf_name in ((1, "model.embed_tokens.weight"), (n_layer + 4, "model.norm.weight"),
                         (n_layer + 5, "lm_head.weight")):
        shards = _read_shards(table[lid], tp_size, lid)
        names = [k for k in shards[0] if "lora_" not in k]
        want = "weight" if lid == n_layer + 4 else "word_embeddings.weight"
        if names != [want]:
            raise ValueError(f"layer {lid}: expected a single tensor {want!r}, found {names}")
        special[hf_name] = list(merge_tensor(want, [s[want] for s in shards]).values())[0]
    emit(special, total)
    vocab = special["lm_head.weight"].shape[0]
    dim = dim or special["model.embed_tokens.weight"].shape[1]
    probe = {}

    def do_block(lid):
        shards = _read_shards(table[lid], tp_size, lid)
        state = {}
        for name in shards[0]:
            if "lora_" in name or name.endswith("rotary_emb.inv_freq"):
                continue
            merged = merge_tensor(name, [s[name] for s in shards], n_heads, num_key_value_heads)
            for k, v in merged.items():
                state[f"model.layers.{lid - 3}.{k}"] = v
        if lid == 3:
            probe.update({k.split(".", 3)[3]: tuple(v.shape) for k, v in state.items()})
        emit(state, lid - 2)

    blocks = [lid for lid in sorted(table) if lid not in (1, n_layer + 4, n_layer + 5)]
    # the first block runs alone so its shapes can fill in missing dimensions
    if blocks:
        if any(PACK.search(n) for n in safe_load(table[blocks[0]][0])) and not (n_heads and num_key_value_heads):
            raise ValueError("packed wqkv checkpoints need --n_heads and --num_key_value_heads")
        do_block(blocks[0])
        with ThreadPoolExecutor(max_workers=workers or int(os.environ.get("LOADWORKER", 8))) as ex:
            list(ex.map(do_block, blocks[1:]))
    index["metadata"] = {"total_size": sum(counts) * 2}
    with open(os.path.join(output_dir, "pytorch_model.bin.index.json"), "w") as f:
        json.dump(index, f, indent=4)

    inter = intermediate_size if intermediate_size and intermediate_size > 0 else \
        probe.get("mlp.gate_proj.weight", (None,))[0]
    q_rows = probe.get("self_attn.q_proj.weight", (dim,))[0]
    k_rows = probe.get("self_attn.k_proj.weight", (dim,))[0]
    n_heads = n_heads or max(1, q_rows // 128)
    head_dim = q_rows // n_heads
    kv = num_key_value_heads if num_key_value_heads and num_key_value_heads > 0 else k_rows // head_dim
    cfg = dict(vocab_size=vocab, hidden_size=dim, intermediate_size=inter, num_attention_heads=n_heads,
               num_key_value_heads=kv, num_hidden_layers=n_layer, rms_norm_eps=norm_eps,
               max_position_embeddings=max_position_embeddings, rope_theta=rope_theta,
               attention_bias="self_attn.q_proj.bias" in probe)
    from transformers import LlamaConfig
    LlamaConfig(**cfg).save_pretrained(output_dir)
    return cfg


def convert_lora(input_dir, output_dir, tp_size=None):
    """peft adapter: ``adapter_model.bin`` with ``base_model.model.…lora_{A,B}.weight`` keys.

    An adapter directory holds files only for the layers that carry adapter tensors (the embedding and head files
    exist only when they are in ``modules_to_save``), so the highest file index says nothing about the depth of the
    model.  A file's role is therefore read from its tensor names: ``word_embeddings.*`` in file 1 is the input
    embedding, in any other file the LM head; everything else is transformer block ``index − 3``."""
    if os.path.abspath(output_dir) == os.path.abspath(input_dir):
        output_dir = os.path.join(output_dir, "convert_hf")
    os.makedirs(output_dir, exist_ok=True)
    table, _ = index_layer_files(input_dir)
    tp_size = tp_size or len(next(iter(table.values())))
    state = {}
    for lid in sorted(table):
        shards = _read_shards(table[lid], tp_size, lid)
        names = list(shards[0])
        if not names or names == ["weight"]:               # the final norm has no adapter
            continue
        embedding_like = all(n.startswith("word_embeddings") for n in names)
        for name in names:
            merged = merge_tensor(name, [s[name] for s in shards])
            for k, v in merged.items():
                if embedding_like and lid == 1:
                    key = k.replace("word_embeddings", "base_model.model.model.embed_tokens")
                    key = key.replace("lora_embedding_A_weight", "lora_embedding_A").replace(
                        "lora_embedding_B_weight", "lora_embedding_B")
                elif embedding_like:
                    key = k.replace("word_embeddings", "base_model.model.lm_head")
                    key = key.replace("lora_embedding_A_weight", "lora_A.weight").replace(
                        "lora_embedding_B_weight", "lora_B.weight")
                else:
                    key = f"base_model.model.model.layers.{lid - 3}.{k}"
                    key = key.replace("lora_A_weight", "lora_A.weight").replace("lora_B_weight", "lora_B.weight")
                state[key] = v
    torch.save(state, os.path.join(output_dir, "adapter_model.bin"))
    src = os.path.join(input_dir, "adapter_config.json")
    if os.path.exists(src):
        shutil.copy(src, os.path.join(output_dir, "adapter_config.json"))
    return sorted(state)
