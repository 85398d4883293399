"""Family ↔ canonical (HF Llama names) state-dict and config translation for ``hf_models``.

The reference vendors one modeling file per family with its own parameter names
(llm/models/hf_models/qwen/modeling_qwen.py ``c_attn`` / ``w1`` / ``w2``, internlm2/modeling_internlm2.py
interleaved ``wqkv``, baichuan*/modeling_baichuan.py ``W_pack``); here one decoder serves all of them and this
module maps their checkpoints in and out."""
from __future__ import annotations

import torch

from ...ckpt.hf_import import canonicalize

_FAMILY_RULES = {"llama": "llama", "internlm": "llama", "baichuan": "baichuan", "baichuan2": "baichuan",
                 "baichuan2-13b": "baichuan", "internlm2": "internlm2", "qwen": "qwen"}


def import_state(hf_state, arch):
    """Any family's on-disk names → ``model.layers.N.self_attn.q_proj.weight`` style names."""
    canon = canonicalize(hf_state, _FAMILY_RULES[arch.family], arch.num_attention_heads, arch.kv_heads, arch.hidden_size)
    out = {}
    for slot, tensors in canon.items():
        for name, t in tensors.items():
            if slot == "embed":
                out["model.embed_tokens.weight"] = t
            elif slot == "norm":
                out["model.norm.weight"] = t
            elif slot == "head":
                out["lm_head.weight"] = t
            else:
                out[f"model.layers.{slot}.{name}"] = t
    return out


def export_state(sd, arch):
    """Canonical names → the family's on-disk names (inverse of ``import_state``)."""
    fam = arch.family
    if fam in ("llama", "internlm"):
        return sd
    out = {}
    L = arch.num_hidden_layers
    hq, hk, d, h = arch.num_attention_heads, arch.kv_heads, arch.head_dim, arch.hidden_size

    def layer(i, name):
        return sd[f"model.layers.{i}.{name}"]
    if fam.startswith("baichuan"):
        for k, v in sd.items():
            if ".self_attn.q_proj." in k or ".self_attn.k_proj." in k or ".self_attn.v_proj." in k:
                continue
            out[k] = v
        for i in range(L):
            out[f"model.layers.{i}.self_attn.W_pack.weight"] = torch.cat(
                [layer(i, f"self_attn.{p}_proj.weight") for p in "qkv"], 0)
        return out
    if fam == "internlm2":
        out["model.tok_embeddings.weight"] = sd["model.embed_tokens.weight"]
        out["model.norm.weight"] = sd["model.norm.weight"]
        out["output.weight"] = sd["lm_head.weight"]
        gs = hq // hk
        for i in range(L):
            q = layer(i, "self_attn.q_proj.weight").view(hk, gs, d, h)
            k = layer(i, "self_attn.k_proj.weight").view(hk, 1, d, h)
            v = layer(i, "self_attn.v_proj.weight").view(hk, 1, d, h)
            out[f"model.layers.{i}.attention.wqkv.weight"] = torch.cat((q, k, v), 1).reshape(-1, h)
            out[f"model.layers.{i}.attention.wo.weight"] = layer(i, "self_attn.o_proj.weight")
            out[f"model.layers.{i}.feed_forward.w1.weight"] = layer(i, "mlp.gate_proj.weight")
            out[f"model.layers.{i}.feed_forward.w3.weight"] = layer(i, "mlp.up_proj.weight")
            out[f"model.layers.{i}.feed_forward.w2.weight"] = layer(i, "mlp.down_proj.weight")
            out[f"model.layers.{i}.attention_norm.weight"] = layer(i, "input_layernorm.weight")
            out[f"model.layers.{i}.ffn_norm.weight"] = layer(i, "post_attention_layernorm.weight")
        return out
    if fam == "qwen":
        out["transformer.wte.weight"] = sd["model.embed_tokens.weight"]
        out["transformer.ln_f.weight"] = sd["model.norm.weight"]
        out["lm_head.weight"] = sd["lm_head.weight"]
        for i in range(L):
            out[f"transformer.h.{i}.attn.c_attn.weight"] = torch.cat([layer(i, f"self_attn.{p}_proj.weight") for p in "qkv"], 0)
            out[f"transformer.h.{i}.attn.c_attn.bias"] = torch.cat([layer(i, f"self_attn.{p}_proj.bias") for p in "qkv"], 0)
            out[f"transformer.h.{i}.attn.c_proj.weight"] = layer(i, "self_attn.o_proj.weight")
            out[f"transformer.h.{i}.mlp.w2.weight"] = layer(i, "mlp.gate_proj.weight")
            out[f"transformer.h.{i}.mlp.w1.weight"] = layer(i, "mlp.up_proj.weight")
            out[f"transformer.h.{i}.mlp.c_proj.weight"] = layer(i, "mlp.down_proj.weight")
            out[f"transformer.h.{i}.ln_1.weight"] = layer(i, "input_layernorm.weight")
            out[f"transformer.h.{i}.ln_2.weight"] = layer(i, "post_attention_layernorm.weight")
        return out
    raise ValueError(fam)


def export_config(arch):
    a = arch
    if a.family == "qwen":
        return {"model_type": "qwen", "vocab_size": a.vocab_size, "hidden_size": a.hidden_size,
                "intermediate_size": 2 * a.intermediate_size, "num_hidden_layers": a.num_hidden_layers,
                "num_attention_heads": a.num_attention_heads, "layer_norm_epsilon": a.rms_norm_eps,
                "rotary_emb_base": a.rope_theta, "use_logn_attn": a.use_logn_attn, "seq_length": a.seq_length,
                "use_cache_quantization": a.use_cache_quantization,
                "use_dynamic_ntk": a.rope_dynamic_ntk_max_pos is not None,
                "max_position_embeddings": a.max_position_embeddings}
    cfg = {"model_type": a.family, "vocab_size": a.vocab_size, "hidden_size": a.hidden_size,
           "intermediate_size": a.intermediate_size, "num_hidden_layers": a.num_hidden_layers,
           "num_attention_heads": a.num_attention_heads, "num_key_value_heads": a.kv_heads,
           "rms_norm_eps": a.rms_norm_eps, "rope_theta": a.rope_theta,
           "max_position_embeddings": a.max_position_embeddings, "tie_word_embeddings": a.tie_word_embeddings,
           "pad_token_id": a.pad_token_id, "bos_token_id": a.bos_token_id, "eos_token_id": a.eos_token_id}
    if a.family in ("internlm", "internlm2"):
        cfg["bias"] = a.qkv_bias
    if a.family == "llama":
        cfg["attention_bias"] = a.qkv_bias
        cfg["architectures"] = ["LlamaForCausalLM"]
    if a.rope_scaling_factor != 1.0:
        cfg["rope_scaling"] = {"type": "dynamic" if a.rope_dynamic_ntk_max_pos else "linear", "factor": a.rope_scaling_factor}
    return cfg
