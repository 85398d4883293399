"""Prompt tuning and prefix tuning on a frozen ``CausalLM``.

The reference's stand-alone fine-tuning script offers these through peft next to LoRA
(llm/runners/open_hf_runner.py:235-623: ``PromptTuningConfig`` / ``PrefixTuningConfig`` branches); here they are two
small wrappers over the package's own decoder:

* ``PromptTuning``: ``num_virtual_tokens`` learnable input embeddings placed in front of every sequence.  The base
  model runs on the concatenated embeddings; labels of the virtual positions are ignored and their logits dropped.
* ``PrefixTuning``: per layer, ``num_virtual_tokens`` learnable key / value vectors every real token can attend to
  (as if the layer's KV cache had been pre-filled).  Token positions start after the prefix, as with a real cache;
  prefix keys are used as stored (no rotary embedding), matching peft's ``past_key_values`` injection.

Only the new tensors train.  ``save_adapter`` / ``load_adapter`` use peft's file names and tensor layout
(``adapter_model.bin`` with ``prompt_embeddings``; for prefixes ``[virtual tokens, layers · 2 · kv_heads · head_dim]``).
"""
from __future__ import annotations

import json
import os

import torch
import torch.nn as nn

from .modeling import build_meta


def _freeze(model):
    for p in model.parameters():
        p.requires_grad_(False)


class PromptTuning(nn.Module):
    def __init__(self, base, num_virtual_tokens=20, init_token_ids=None):
        super().__init__()
        _freeze(base)
        self.base, self.n = base, int(num_virtual_tokens)
        emb = base.get_input_embeddings()
        if init_token_ids is not None:           # peft's TEXT init: repeat / cut the tokenised text to n tokens
            ids = torch.as_tensor(list(init_token_ids), dtype=torch.long, device=emb.weight.device)
            ids = ids.repeat((self.n + len(ids) - 1) // len(ids))[:self.n]
            init = emb(ids).detach().clone()
        else:
            init = torch.randn(self.n, emb.weight.shape[1], dtype=emb.weight.dtype, device=emb.weight.device) * 0.02
        self.prompt_embeddings = nn.Parameter(init.float())
        self.arch = self.config = base.arch

    def forward(self, input_ids, attention_mask=None, labels=None, **kw):
        b, s = input_ids.shape
        emb = self.base.get_input_embeddings()(input_ids)
        x = torch.cat((self.prompt_embeddings.to(emb.dtype).unsqueeze(0).expand(b, -1, -1), emb), dim=1)
        ids = torch.cat((input_ids.new_zeros(b, self.n), input_ids), dim=1)          # shapes / metadata only
        mask = torch.ones(b, s, dtype=torch.long, device=input_ids.device) if attention_mask is None else attention_mask
        mask = torch.cat((mask.new_ones(b, self.n), mask), dim=1)
        if labels is not None:
            labels = torch.cat((labels.new_full((b, self.n), -100), labels), dim=1)
        out = self.base(ids, mask, labels=labels, inputs_embeds=x, **kw)
        if "logits" in out:
            out["logits"] = out["logits"][:, self.n:]
        return out

    def generate(self, input_ids, **kw):
        return self.base.generate(input_ids, soft_prefix={"embeds": self.prompt_embeddings.detach()}, **kw)

    def generate_stream(self, input_ids, **kw):
        return self.base.generate_stream(input_ids, soft_prefix={"embeds": self.prompt_embeddings.detach()}, **kw)

    def adapter_state(self):
        return {"prompt_embeddings": self.prompt_embeddings.detach().cpu()}

    def adapter_config(self):
        a = self.arch
        return {"peft_type": "PROMPT_TUNING", "task_type": "CAUSAL_LM", "num_virtual_tokens": self.n,
                "token_dim": a.hidden_size, "num_layers": a.num_hidden_layers,
                "num_attention_heads": a.num_attention_heads, "num_transformer_submodules": 1, "inference_mode": True}

    def load_adapter_state(self, sd):
        self.prompt_embeddings.data.copy_(sd["prompt_embeddings"].to(self.prompt_embeddings))


class PrefixTuning(nn.Module):
    def __init__(self, base, num_virtual_tokens=20):
        super().__init__()
        _freeze(base)
        a = base.arch
        self.base, self.n, self.arch, self.config = base, int(num_virtual_tokens), a, a
        dev = base.get_input_embeddings().weight.device
        # [layers, key|value, virtual tokens, kv heads, head dim]
        self.prefix = nn.Parameter(torch.randn(a.num_hidden_layers, 2, self.n, a.kv_heads, a.head_dim, device=dev) * 0.02)

    def forward(self, input_ids, attention_mask=None, labels=None, **_):
        from ... import ops
        a, base = self.arch, self.base
        b, s = input_ids.shape
        dt = base.lm_head.weight.dtype
        pos = (torch.arange(s, device=input_ids.device) + self.n).unsqueeze(0).expand(b, s)
        meta = build_meta(input_ids, None, pos)
        caches = []
        for l in range(a.num_hidden_layers):
            kv = self.prefix[l].to(dt).unsqueeze(1).expand(2, b, self.n, a.kv_heads, a.head_dim)
            room = kv.new_zeros(2, b, s, a.kv_heads, a.head_dim)
            full = torch.cat((kv, room), dim=2)
            caches.append({"k": full[0], "v": full[1], "len": self.n})
        h = base.hidden_states(input_ids, meta, caches)
        out = {}
        if labels is not None:
            shift = torch.full_like(labels, -100)
            shift[:, :-1] = labels[:, 1:]
            if attention_mask is not None:
                shift = shift.masked_fill(attention_mask == 0, -100)
            flat = shift.reshape(-1)
            valid = flat != -100
            tok = ops.lm_head_cross_entropy(h, base.head_weight(), flat.masked_fill(~valid, 0))
            out["loss"] = (tok * valid).sum() / valid.sum().clamp(min=1)
            out["num_tokens"] = valid.sum().detach()
        else:
            out["logits"] = ops.linear(h, base.head_weight()).view(b, s, -1)
        return out

    def generate(self, input_ids, **kw):
        return self.base.generate(input_ids, soft_prefix={"kv": self.prefix.detach()}, **kw)

    def generate_stream(self, input_ids, **kw):
        return self.base.generate_stream(input_ids, soft_prefix={"kv": self.prefix.detach()}, **kw)

    def adapter_state(self):
        L, _, P, hk, d = self.prefix.shape
        return {"prompt_embeddings": self.prefix.detach().permute(2, 0, 1, 3, 4).reshape(P, L * 2 * hk * d).cpu()}

    def adapter_config(self):
        a = self.arch
        return {"peft_type": "PREFIX_TUNING", "task_type": "CAUSAL_LM", "num_virtual_tokens": self.n,
                "token_dim": a.kv_heads * a.head_dim, "num_layers": a.num_hidden_layers,
                "num_attention_heads": a.kv_heads, "num_transformer_submodules": 1, "prefix_projection": False,
                "inference_mode": True}

    def load_adapter_state(self, sd):
        L, _, P, hk, d = self.prefix.shape
        t = sd["prompt_embeddings"].reshape(P, L, 2, hk, d).permute(1, 2, 0, 3, 4)
        self.prefix.data.copy_(t.to(self.prefix))


def save_adapter(model, out_dir, config_name="adapter_config.json"):
    os.makedirs(out_dir, exist_ok=True)
    torch.save(model.adapter_state(), os.path.join(out_dir, "adapter_model.bin"))
    with open(os.path.join(out_dir, config_name), "w") as f:
        json.dump(model.adapter_config(), f, indent=2)


def load_adapter(base, adapter_dir, config_name="adapter_config.json"):
    """Wrap ``base`` with the tuning method recorded in ``adapter_dir`` and load its tensors."""
    with open(os.path.join(adapter_dir, config_name)) as f:
        cfg = json.load(f)
    kind = cfg.get("peft_type")
    if kind == "PROMPT_TUNING":
        m = PromptTuning(base, cfg["num_virtual_tokens"])
    elif kind == "PREFIX_TUNING":
        m = PrefixTuning(base, cfg["num_virtual_tokens"])
    else:
        raise ValueError(f"{adapter_dir}: unsupported peft_type {kind!r}")
    m.load_adapter_state(torch.load(os.path.join(adapter_dir, "adapter_model.bin"), map_location="cpu"))
    return m
