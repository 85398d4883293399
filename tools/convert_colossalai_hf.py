"""ColossalAI pipeline/tensor-parallel Llama shards → HuggingFace checkpoint
(tools/convert_colossalai_hf.py:103-357 of the reference).

    python tools/convert_colossalai_hf.py --input_dir shards --output_dir hf --n_heads 32 --dim 4096 [--tp_size 2]

Shard files ``*tp{t}_pp{p}*.pt`` (or ``.bin``) hold names like ``model.layers.N.attention.wq.weight``
with layer numbers local to their pipeline stage.  Stages are concatenated in order, TP shards are
merged (column-parallel: rows; row-parallel: columns; norms: first shard), and the interleaved
rotary layout of q/k is permuted to HF's half-rotation layout.
"""
import argparse
import glob
import json
import os
import re
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

COL = ("wq", "wk", "wv", "w1", "w3", "tok_embeddings", "output")
ROW = ("wo", "w2")
NAME = {"attention.wq": "self_attn.q_proj", "attention.wk": "self_attn.k_proj", "attention.wv": "self_attn.v_proj",
        "attention.wo": "self_attn.o_proj", "feed_forward.w1": "mlp.gate_proj", "feed_forward.w3": "mlp.up_proj",
        "feed_forward.w2": "mlp.down_proj", "attention_norm": "input_layernorm", "ffn_norm": "post_attention_layernorm"}


def permute_rope(w, n_heads, dim_out, dim_in):
    """Interleaved (x0,x1,x2,…) rotary pairs → HF half layout."""
    return w.view(n_heads, dim_out // n_heads // 2, 2, dim_in).transpose(1, 2).reshape(dim_out, dim_in)


def merge(name, shards):
    if any(k in name for k in COL):
        return torch.cat(shards, 0)
    if any(k in name for k in ROW):
        return torch.cat(shards, 1)
    return shards[0]


def main(argv=None):
    p = argparse.ArgumentParser()
    p.add_argument("--input_dir", required=True)
    p.add_argument("--output_dir", required=True)
    p.add_argument("--n_heads", type=int, required=True)
    p.add_argument("--n_kv_heads", type=int, default=None)
    p.add_argument("--dim", type=int, required=True)
    p.add_argument("--norm_eps", type=float, default=1e-6)
    a = p.parse_args(argv)
    files = {}
    for f in glob.glob(os.path.join(a.input_dir, "*")):
        m = re.search(r"tp(\d+)_pp(\d+)", os.path.basename(f))
        if m:
            files[(int(m.group(2)), int(m.group(1)))] = f
    if not files:
        raise SystemExit("no *tp{t}_pp{p}* shard files found")
    pps, tps = sorted({k[0] for k in files}), sorted({k[1] for k in files})
    out, layer_base = {}, 0
    for pp in pps:
        shards = [torch.load(files[(pp, tp)], map_location="cpu") for tp in tps]
        local_layers = 0
        for name in shards[0]:
            t = merge(name, [s[name] for s in shards])
            m = re.match(r"(?:model\.)?layers\.(\d+)\.(.+)\.weight$", name)
            if m:
                li, sub = int(m.group(1)), m.group(2)
                local_layers = max(local_layers, li + 1)
                if sub in ("attention.wq", "attention.wk"):
                    heads = a.n_heads if sub.endswith("wq") else (a.n_kv_heads or a.n_heads)
                    t = permute_rope(t, heads, t.shape[0], t.shape[1])
                out[f"model.layers.{layer_base + li}.{NAME[sub]}.weight"] = t
            elif "tok_embeddings" in name:
                out["model.embed_tokens.weight"] = t
            elif name.endswith("output.weight"):
                out["lm_head.weight"] = t
            elif name.endswith("norm.weight"):
                out["model.norm.weight"] = t
        layer_base += local_layers
    os.makedirs(a.output_dir, exist_ok=True)
    torch.save(out, os.path.join(a.output_dir, "pytorch_model.bin"))
    inter = out["model.layers.0.mlp.gate_proj.weight"].shape[0]
    cfg = {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_size": a.dim,
           "intermediate_size": inter, "num_attention_heads": a.n_heads,
           "num_key_value_heads": a.n_kv_heads or a.n_heads, "num_hidden_layers": layer_base,
           "rms_norm_eps": a.norm_eps, "vocab_size": out["model.embed_tokens.weight"].shape[0]}
    with open(os.path.join(a.output_dir, "config.json"), "w") as f:
        json.dump(cfg, f, indent=2)
    print(f"wrote {layer_base} layers to {a.output_dir}")


if __name__ == "__main__":
    main()
