"""HuggingFace-format weights → this framework's TP-sharded layers.

Parity: llm/models/mg_models/llama/utils.py:58-350 — family name maps (Llama; Qwen v1:
``c_attn`` split, ``w2→gate``, ``w1→up``; InternLM2: ``wqkv`` de-interleaved by GQA group,
``w1/w3/w2 → gate/up/down``; Baichuan ``W_pack``), TP slicing on load (column-parallel:
rows, row-parallel: columns, vocab: rows; q/k/v sliced separately then fused), ``.bin`` /
``.safetensors`` shards, vocab padding when the tokenizer was extended.

Instead of one if-chain per family the map is a regex rule table producing a canonical
per-layer dict (the names stored in layer files); slicing is decided by the destination
parameter's ``partition_dim`` tag, not by name lists.
"""
from __future__ import annotations

import glob
import json
import os
import re
from concurrent.futures import ThreadPoolExecutor
from typing import Dict

import torch

from ..parallel.grid import get_grid
from ..utils.log import default_logger as logger

# (regex on the HF key) -> canonical "<layer|embed|norm|head>:<name>"
_LLAMA_RULES = [
    (r"^model\.embed_tokens\.weight$", "embed:word_embeddings.weight"),
    (r"^model\.norm\.weight$", "norm:weight"),
    (r"^lm_head\.weight$", "head:word_embeddings.weight"),
    (r"^model\.layers\.(\d+)\.(self_attn\.(?:q|k|v|o)_proj\.(?:weight|bias))$", r"\1:\2"),
    (r"^model\.layers\.(\d+)\.(mlp\.(?:gate|up|down)_proj\.weight)$", r"\1:\2"),
    (r"^model\.layers\.(\d+)\.((?:input|post_attention)_layernorm\.weight)$", r"\1:\2"),
    (r"^model\.layers\.(\d+)\.self_attn\.W_pack\.weight$", r"\1:@wpack"),
]
_QWEN_RULES = [
    (r"^transformer\.wte\.weight$", "embed:word_embeddings.weight"),
    (r"^transformer\.ln_f\.weight$", "norm:weight"),
    (r"^lm_head\.weight$", "head:word_embeddings.weight"),
    (r"^transformer\.h\.(\d+)\.attn\.c_attn\.(weight|bias)$", r"\1:@c_attn.\2"),
    (r"^transformer\.h\.(\d+)\.attn\.c_proj\.weight$", r"\1:self_attn.o_proj.weight"),
    (r"^transformer\.h\.(\d+)\.mlp\.w2\.weight$", r"\1:mlp.gate_proj.weight"),
    (r"^transformer\.h\.(\d+)\.mlp\.w1\.weight$", r"\1:mlp.up_proj.weight"),
    (r"^transformer\.h\.(\d+)\.mlp\.c_proj\.weight$", r"\1:mlp.down_proj.weight"),
    (r"^transformer\.h\.(\d+)\.ln_1\.weight$", r"\1:input_layernorm.weight"),
    (r"^transformer\.h\.(\d+)\.ln_2\.weight$", r"\1:post_attention_layernorm.weight"),
]
_INTERNLM2_RULES = [
    (r"^model\.tok_embeddings\.weight$", "embed:word_embeddings.weight"),
    (r"^model\.norm\.weight$", "norm:weight"),
    (r"^output\.weight$", "head:word_embeddings.weight"),
    (r"^model\.layers\.(\d+)\.attention\.wqkv\.weight$", r"\1:@wqkv_grouped"),
    (r"^model\.layers\.(\d+)\.attention\.wo\.weight$", r"\1:self_attn.o_proj.weight"),
    (r"^model\.layers\.(\d+)\.feed_forward\.w1\.weight$", r"\1:mlp.gate_proj.weight"),
    (r"^model\.layers\.(\d+)\.feed_forward\.w3\.weight$", r"\1:mlp.up_proj.weight"),
    (r"^model\.layers\.(\d+)\.feed_forward\.w2\.weight$", r"\1:mlp.down_proj.weight"),
    (r"^model\.layers\.(\d+)\.attention_norm\.weight$", r"\1:input_layernorm.weight"),
    (r"^model\.layers\.(\d+)\.ffn_norm\.weight$", r"\1:post_attention_layernorm.weight"),
]
RULES = {"llama": _LLAMA_RULES, "llama_pack": _LLAMA_RULES, "qwen": _QWEN_RULES,
         "internlm2": _INTERNLM2_RULES, "internlm2_pack": _INTERNLM2_RULES, "baichuan": _LLAMA_RULES,
         "internlm": _LLAMA_RULES}


def canonicalize(hf_state: Dict[str, torch.Tensor], pretrain_type: str, n_heads: int, n_kv_heads: int,
                 hidden: int) -> Dict[str, Dict[str, torch.Tensor]]:
    """HF state dict → {slot: {canonical name: full tensor}}; slot is 'embed' | 'norm' | 'head' |
    '<layer number>'.  Packed projections are split into q/k/v here."""
    rules = [(re.compile(p), r) for p, r in RULES[pretrain_type]]
    out: Dict[str, Dict[str, torch.Tensor]] = {}
    head_dim = hidden // n_heads
    for key, t in hf_state.items():
        target = None
        for pat, repl in rules:
            m = pat.match(key)
            if m:
                target = m.expand(repl)
                break
        if target is None:
            if "rotary_emb.inv_freq" not in key:
                logger.info(f"unused key {key}")
            continue
        slot, name = target.split(":", 1)
        d = out.setdefault(slot, {})
        if name.startswith("@c_attn") or name == "@wpack":
            kind = name.split(".")[-1] if "." in name else "weight"
            q, k, v = torch.chunk(t, 3, dim=0)
            for n, part in (("q", q), ("k", k), ("v", v)):
                d[f"self_attn.{n}_proj.{kind}"] = part.contiguous()
        elif name == "@wqkv_grouped":
            gs = n_heads // n_kv_heads
            w = t.reshape(-1, gs + 2, head_dim, hidden)
            d["self_attn.q_proj.weight"] = w[:, :gs].reshape(-1, hidden).contiguous()
            d["self_attn.k_proj.weight"] = w[:, -2].reshape(-1, hidden).contiguous()
            d["self_attn.v_proj.weight"] = w[:, -1].reshape(-1, hidden).contiguous()
        else:
            d[name] = t
    return out


def load_hf_state(path, worker=8):
    """Read every weight shard under ``path`` (index json, ``*.safetensors`` or ``*.bin``)."""
    files = []
    for idx in ("model.safetensors.index.json", "pytorch_model.bin.index.json"):
        p = os.path.join(path, idx)
        if os.path.exists(p):
            with open(p) as f:
                files = sorted(set(json.load(f)["weight_map"].values()))
            break
    if not files:
        files = sorted(os.path.basename(p) for p in glob.glob(os.path.join(path, "*.safetensors"))) or \
            sorted(os.path.basename(p) for p in glob.glob(os.path.join(path, "pytorch_model*.bin")))
    if not files:
        raise FileNotFoundError(f"no HF weight files under {path}")

    def read(fn):
        fp = os.path.join(path, fn)
        if fn.endswith(".safetensors"):
            from safetensors.torch import load_file
            return load_file(fp)
        return torch.load(fp, map_location="cpu", weights_only=False)

    state = {}
    with ThreadPoolExecutor(max_workers=max(1, worker)) as ex:
        for part in ex.map(read, files):
            state.update(part)
    return state


def _slice_for(param, full, tp, rank):
    dim = getattr(param, "partition_dim", -1)
    if not getattr(param, "tensor_model_parallel", False) or tp == 1 or dim < 0:
        return full
    n = full.shape[dim] // tp
    return full.narrow(dim, rank * n, n)


def load_canonical_into_model(model, canon, pad_vocab=True):
    """Copy canonical full tensors into this rank's (TP-sliced, fused) parameters."""
    g = get_grid()
    L = model.num_layers
    slot_of = {1: "embed", L + 4: "norm", L + 5: "head"}
    loaded = 0
    with torch.no_grad():
        for key, mod in model.layers.items():
            idx = int(key)
            src = canon.get(slot_of.get(idx, str(idx - 3)))
            if src is None:
                raise KeyError(f"no weights for layer index {idx}")
            sd = {}
            for name, full in src.items():
                sd[name] = full
            if idx in (1, L + 5):
                w = sd["word_embeddings.weight"]
                V = mod.word_embeddings.num_embeddings
                if w.shape[0] < V and pad_vocab:       # tokenizer was extended: pad with the mean row
                    pad = w.mean(0, keepdim=True).expand(V - w.shape[0], -1)
                    w = torch.cat((w, pad.to(w.dtype)), 0)
                elif w.shape[0] > V:
                    w = w[:V]
                sd["word_embeddings.weight"] = w
            # slice every tensor for this TP rank using the reference (unfused) names
            sliced = {}
            for name, full in sd.items():
                sliced[name] = _tp_slice_by_name(name, full, g.tp, g.tp_rank)
            missing, unexpected = mod.load_state_dict({k: v.to(next(mod.parameters()).dtype) for k, v in sliced.items()},
                                                      strict=False)
            missing = [m for m in missing if "lora_" not in m]
            if missing or unexpected:
                raise RuntimeError(f"layer {idx}: missing {missing}, unexpected {unexpected}")
            loaded += len(sliced)
    return loaded


_COL = re.compile(r"(q_proj|k_proj|v_proj|gate_proj|up_proj)\.(weight|bias)$|word_embeddings\.weight$")
_ROW = re.compile(r"(o_proj|down_proj)\.weight$")


def _tp_slice_by_name(name, full, tp, rank):
    if tp == 1:
        return full
    if _COL.search(name):
        n = full.shape[0] // tp
        return full.narrow(0, rank * n, n)
    if _ROW.search(name):
        n = full.shape[1] // tp
        return full.narrow(1, rank * n, n)
    return full


def load_llama_from_hf_format(model, load_path, pretrain_type="llama", worker=8, debug=False):
    """Entry used by the checkpoint helper's ``load_mode: huggingface``."""
    if debug:
        logger.info("loader.debug: skipping weight loading")
        return 0
    a = model.args
    state = load_hf_state(load_path, worker)
    canon = canonicalize(state, pretrain_type, a.num_attention_heads, a.num_kv_attention_heads, a.hidden_size)
    return load_canonical_into_model(model, canon)
