"""HuggingFace-style causal LMs for the data-parallel runner: one decoder, many families.

The reference vendors ~14 kLoC of per-family remote code patched to call flash-attn
(llm/models/hf_models/{llama,internlm,internlm2,baichuan,baichuan2,qwen}/modeling_*.py,
utils/flash_utils.py:62-655).  Here every family is one ``CausalLM`` parameterised by an
``HFArch`` record (RoPE vs ALiBi, q/k/v/o biases, GQA, norm-head, NTK / log-n scaling) that runs
on this framework's kernels: fused RMSNorm, RoPE on the packed QKV rows, causal segment-aware
flash attention (``cu_seqlens`` packing; padding is expressed as extra segments), SwiGLU and
the fused LM-head cross-entropy.  Checkpoints keep each family's own tensor names on disk
(``from_pretrained`` / ``save_pretrained`` translate through ``ckpt.hf_import`` rules).

Module attribute names follow HF Llama (``model.layers[i].self_attn`` …) so tools that walk the
module tree (Dynamic Checkpoint's ``level_keys: layers``, LoRA target names) work unchanged.
"""
from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ... import ops
from ...ops import reference as ref
from ..layers import RotaryTables, alibi_slopes


@dataclass
class HFArch:
    family: str = "llama"                 # llama | internlm | internlm2 | baichuan | baichuan2 | baichuan2-13b | qwen
    vocab_size: int = 32000
    hidden_size: int = 4096
    intermediate_size: int = 11008
    num_hidden_layers: int = 32
    num_attention_heads: int = 32
    num_key_value_heads: Optional[int] = None
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    rope_scaling_factor: float = 1.0
    rope_dynamic_ntk_max_pos: Optional[int] = None
    max_position_embeddings: int = 4096
    qkv_bias: bool = False
    o_bias: bool = False
    position: str = "rope"                # rope | alibi
    norm_head: bool = False               # Baichuan2: rows of lm_head are L2-normalised
    use_logn_attn: bool = False           # Qwen inference-time log-n scaling of queries
    use_cache_quantization: bool = False  # Qwen: keep the decode KV cache in uint8 (per-chunk scale / zero)
    seq_length: int = 2048                # Qwen: training length for log-n / NTK
    tie_word_embeddings: bool = False
    pad_token_id: Optional[int] = None
    bos_token_id: Optional[int] = 1
    eos_token_id: Optional[int] = 2

    @property
    def kv_heads(self):
        return self.num_key_value_heads or self.num_attention_heads

    @property
    def head_dim(self):
        return self.hidden_size // self.num_attention_heads


def arch_from_hf_config(cfg: dict, family: Optional[str] = None) -> HFArch:
    """Translate a family's ``config.json`` into an HFArch."""
    mt = (family or cfg.get("model_type") or "llama").lower()
    a = HFArch(family=mt)
    g = cfg.get
    if mt == "qwen":
        a.vocab_size, a.hidden_size = g("vocab_size"), g("hidden_size")
        a.intermediate_size = g("intermediate_size", 4 * a.hidden_size) // 2   # Qwen stores 2·ffn
        a.num_hidden_layers, a.num_attention_heads = g("num_hidden_layers"), g("num_attention_heads")
        a.rms_norm_eps = g("layer_norm_epsilon", 1e-6)
        a.rope_theta = g("rotary_emb_base", 10000.0)
        a.qkv_bias, a.use_logn_attn, a.seq_length = True, g("use_logn_attn", False), g("seq_length", 2048)
        a.use_cache_quantization = bool(g("use_cache_quantization", False))
        a.rope_dynamic_ntk_max_pos = a.seq_length if g("use_dynamic_ntk", False) else None
        a.max_position_embeddings = g("max_position_embeddings", 8192)
        return a
    a.vocab_size, a.hidden_size = g("vocab_size", 32000), g("hidden_size", 4096)
    a.intermediate_size = g("intermediate_size", 11008)
    a.num_hidden_layers, a.num_attention_heads = g("num_hidden_layers", 32), g("num_attention_heads", 32)
    a.num_key_value_heads = g("num_key_value_heads")
    a.rms_norm_eps = g("rms_norm_eps", 1e-6)
    a.rope_theta = g("rope_theta", 10000.0)
    a.max_position_embeddings = g("max_position_embeddings", g("model_max_length", 4096))
    sc = g("rope_scaling") or {}
    if sc.get("type") == "linear":
        a.rope_scaling_factor = float(sc.get("factor", 1.0))
    elif sc.get("type") == "dynamic":
        a.rope_scaling_factor, a.rope_dynamic_ntk_max_pos = float(sc.get("factor", 1.0)), a.max_position_embeddings
    a.tie_word_embeddings = g("tie_word_embeddings", False)
    a.pad_token_id, a.bos_token_id, a.eos_token_id = g("pad_token_id"), g("bos_token_id", 1), g("eos_token_id", 2)
    if mt in ("internlm",):
        a.qkv_bias = a.o_bias = g("bias", True)
    if mt == "internlm2":
        a.qkv_bias = a.o_bias = g("bias", False)
    if mt in ("llama",):
        a.qkv_bias = a.o_bias = g("attention_bias", False)
    if mt.startswith("baichuan2"):
        a.norm_head = True
    if mt == "baichuan2-13b" or (mt.startswith("baichuan") and a.num_hidden_layers >= 40):
        a.position, a.family = "alibi", "baichuan2-13b" if mt.startswith("baichuan2") else mt
    return a


class RMSNorm(nn.Module):
    def __init__(self, dim, eps, dtype):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim, dtype=dtype))
        self.eps = eps

    def forward(self, x, residual=None):
        if residual is None:
            return ops.rmsnorm(x, self.weight, self.eps)
        return ops.add_rmsnorm(x, residual, self.weight, self.eps)


class Attention(nn.Module):
    def __init__(self, a: HFArch, dtype):
        super().__init__()
        self.a = a
        d, hq, hk = a.head_dim, a.num_attention_heads, a.kv_heads
        self.q_proj = nn.Linear(a.hidden_size, hq * d, bias=a.qkv_bias, dtype=dtype)
        self.k_proj = nn.Linear(a.hidden_size, hk * d, bias=a.qkv_bias, dtype=dtype)
        self.v_proj = nn.Linear(a.hidden_size, hk * d, bias=a.qkv_bias, dtype=dtype)
        self.o_proj = nn.Linear(hq * d, a.hidden_size, bias=a.o_bias, dtype=dtype)
        self.rotary = RotaryTables(d, a.rope_theta, a.rope_scaling_factor, a.rope_dynamic_ntk_max_pos) \
            if a.position == "rope" else None
        self.slopes = torch.tensor(alibi_slopes(hq), dtype=torch.float32) if a.position == "alibi" else None

    def forward(self, x, meta, cache=None):
        a = self.a
        d, hq, hk = a.head_dim, a.num_attention_heads, a.kv_heads
        T = x.shape[0]
        qkv = ops.linear_parts(x, (self.q_proj.weight, self.k_proj.weight, self.v_proj.weight),
                               (self.q_proj.bias, self.k_proj.bias, self.v_proj.bias) if a.qkv_bias else None)
        pos = meta["position_ids"]
        rope = None
        if self.rotary is not None:
            cos, sin = self.rotary.get(int(meta["max_position"]), x.device)
            rope = (cos, sin, pos)
        if cache is None and not (a.use_logn_attn and not self.training):
            # training / full-sequence path: RoPE + attention on the packed projection, one packed gradient back
            sl = self.slopes.to(x.device) if self.slopes is not None else None
            o = ops.flash_attention_packed(qkv, hq, hk, d, meta["cu_seqlens"], meta["max_seqlen"], alibi_slopes=sl,
                                           rope=rope, row_start=meta.get("row_start"))
            return ops.linear(o, self.o_proj.weight, self.o_proj.bias)
        if rope is not None:
            qkv = ops.rope_packed(qkv, cos, sin, pos, hq, hk, d)
        q = qkv[:, :hq * d].view(T, hq, d)
        k = qkv[:, hq * d:(hq + hk) * d].view(T, hk, d)
        v = qkv[:, (hq + hk) * d:].view(T, hk, d)
        if a.use_logn_attn and not self.training:
            logn = torch.clamp(torch.log(pos.float() + 1) / math.log(a.seq_length), min=1.0)
            q = (q.float() * logn.view(T, 1, 1)).to(q.dtype)
        if cache is not None:
            B = meta["batch"]
            S = T // B
            p0 = cache["len"]
            cache_ref = cache
            if "kq" in cache:                 # 8-bit cache: quantise the new chunk, attend over the dequantised prefix
                cache["kq"].append(p0, k.reshape(B, S, hk, d))
                cache["vq"].append(p0, v.reshape(B, S, hk, d))
                cache = dict(cache, k=cache["kq"].read(p0 + S), v=cache["vq"].read(p0 + S))
                cache_ref["len"] = p0 + S
            else:
                cache["k"][:, p0:p0 + S] = k.reshape(B, S, hk, d)
                cache["v"][:, p0:p0 + S] = v.reshape(B, S, hk, d)
                cache["len"] = p0 + S
            if meta.get("tree_mask") is not None:
                o = _tree_cached(q.reshape(B, S, hq, d), cache["k"][:, :p0 + S], cache["v"][:, :p0 + S], p0,
                                 meta["tree_mask"])
            elif self.slopes is not None:
                o = _alibi_cached(q.reshape(B, S, hq, d), cache["k"][:, :p0 + S], cache["v"][:, :p0 + S], p0,
                                  self.slopes.to(x.device))
            else:
                o = ref.attention_kvcache(q.reshape(B, S, hq, d), cache["k"][:, :p0 + S], cache["v"][:, :p0 + S], p0)
            o = o.reshape(T, hq * d)
        else:
            sl = self.slopes.to(x.device) if self.slopes is not None else None
            o = ops.flash_attention(q, k, v, meta["cu_seqlens"], meta["max_seqlen"], True, alibi_slopes=sl)
            o = o.reshape(T, hq * d)
        return ops.linear(o, self.o_proj.weight, self.o_proj.bias)


def _tree_cached(q, kc, vc, p0, tree_mask):
    """Speculative-tree attention: every draft node sees the whole prefix cache and its ancestors."""
    B, Sq, H, D = q.shape
    rep = H // kc.shape[2]
    s = torch.einsum("bqhd,bkhd->bhqk", q.float(), kc.float().repeat_interleave(rep, 2)) / math.sqrt(D)
    full = torch.ones(Sq, p0 + Sq, dtype=torch.bool, device=q.device)
    full[:, p0:] = tree_mask
    s = s.masked_fill(~full.view(1, 1, Sq, p0 + Sq), float("-inf"))
    return torch.einsum("bhqk,bkhd->bqhd", torch.softmax(s, -1), vc.float().repeat_interleave(rep, 2)).to(q.dtype)


def _alibi_cached(q, kc, vc, p0, slopes):
    B, Sq, H, D = q.shape
    Sk = kc.shape[1]
    rep = H // kc.shape[2]
    s = torch.einsum("bqhd,bkhd->bhqk", q.float(), kc.float().repeat_interleave(rep, 2)) / math.sqrt(D)
    qi = torch.arange(Sq, device=q.device).view(Sq, 1) + p0
    kj = torch.arange(Sk, device=q.device).view(1, Sk)
    s = s + slopes.view(1, H, 1, 1) * (kj - qi).view(1, 1, Sq, Sk)
    s = s.masked_fill((kj > qi).view(1, 1, Sq, Sk), float("-inf"))
    return torch.einsum("bhqk,bkhd->bqhd", torch.softmax(s, -1), vc.float().repeat_interleave(rep, 2)).to(q.dtype)


class MLP(nn.Module):
    def __init__(self, a: HFArch, dtype):
        super().__init__()
        self.gate_proj = nn.Linear(a.hidden_size, a.intermediate_size, bias=False, dtype=dtype)
        self.up_proj = nn.Linear(a.hidden_size, a.intermediate_size, bias=False, dtype=dtype)
        self.down_proj = nn.Linear(a.intermediate_size, a.hidden_size, bias=False, dtype=dtype)

    def forward(self, x):
        gu = ops.linear_parts(x, (self.gate_proj.weight, self.up_proj.weight))
        return ops.linear(ops.glu(gu, "silu"), self.down_proj.weight)


class DecoderLayer(nn.Module):
    def __init__(self, a: HFArch, dtype):
        super().__init__()
        self.self_attn = Attention(a, dtype)
        self.mlp = MLP(a, dtype)
        self.input_layernorm = RMSNorm(a.hidden_size, a.rms_norm_eps, dtype)
        self.post_attention_layernorm = RMSNorm(a.hidden_size, a.rms_norm_eps, dtype)

    def forward(self, delta, residual, meta, cache=None):
        if residual is None:
            h = delta
            n1 = self.input_layernorm(h)
        else:
            n1, h = self.input_layernorm(delta, residual)
        n2, h = self.post_attention_layernorm(self.self_attn(n1, meta, cache), h)
        return self.mlp(n2), h


class Decoder(nn.Module):
    def __init__(self, a: HFArch, dtype):
        super().__init__()
        self.embed_tokens = nn.Embedding(a.vocab_size, a.hidden_size, dtype=dtype)
        self.layers = nn.ModuleList(DecoderLayer(a, dtype) for _ in range(a.num_hidden_layers))
        self.norm = RMSNorm(a.hidden_size, a.rms_norm_eps, dtype)


def build_meta(input_ids, attention_mask=None, position_ids=None, cu_seqlens=None, device=None):
    """Token-major metadata.  Padding becomes its own segments so real tokens never see it.
    Everything is computed where ``input_ids`` lives and then moved to ``device``: with a batch still on the host
    (as a loader delivers it) the scalars below cost no device→host synchronisation."""
    b, s = input_ids.shape
    dev = input_ids.device
    out_dev = torch.device(device) if device is not None else dev
    if cu_seqlens is not None:
        cu = torch.unique_consecutive(cu_seqlens.reshape(-1).to(torch.int32))
        if int(cu[-1]) < b * s:
            cu = torch.cat((cu, cu.new_tensor([b * s])))
    else:
        bounds = set(range(0, (b + 1) * s, s))
        if attention_mask is not None and not bool(attention_mask.all()):
            m = attention_mask.bool()
            for i in range(b):
                edges = torch.nonzero(m[i, 1:] != m[i, :-1]).flatten() + 1
                bounds.update(i * s + int(e) for e in edges)
        cu = torch.tensor(sorted(bounds), dtype=torch.int32, device=dev)
    if position_ids is None:
        if attention_mask is not None and not bool(attention_mask.all()):
            position_ids = (attention_mask.long().cumsum(-1) - 1).clamp(min=0)
        else:
            position_ids = torch.arange(s, device=dev).unsqueeze(0).expand(b, s)
    pos = position_ids.reshape(-1).to(torch.int32)
    meta = {"max_seqlen": int((cu[1:] - cu[:-1]).max()), "batch": b, "max_position": max(s, int(pos.max()) + 1)}
    row_start = None
    if out_dev.type == "cuda":
        from ...ops import cuda as cu_ops
        if cu_ops.available():
            row_start = cu_ops.row_start_of(cu, b * s, out_dev)   # once per batch, not once per layer
    meta.update(position_ids=pos.to(out_dev, non_blocking=True), cu_seqlens=cu.to(out_dev, non_blocking=True),
                row_start=row_start)
    return meta


class CausalLM(nn.Module):
    def __init__(self, arch: HFArch, dtype=torch.float32):
        super().__init__()
        self.arch = arch
        self.config = arch
        self.model = Decoder(arch, dtype)
        self.lm_head = nn.Linear(arch.hidden_size, arch.vocab_size, bias=False, dtype=dtype)
        self.gradient_checkpointing = False
        self.apply(self._init)

    @staticmethod
    def _init(m):
        if isinstance(m, (nn.Linear, nn.Embedding)):
            nn.init.normal_(m.weight, 0.0, 0.02)
            if getattr(m, "bias", None) is not None:
                nn.init.zeros_(m.bias)

    def gradient_checkpointing_enable(self, **_):
        self.gradient_checkpointing = True

    def gradient_checkpointing_disable(self):
        self.gradient_checkpointing = False

    def get_input_embeddings(self):
        return self.model.embed_tokens

    def head_weight(self):
        w = self.lm_head.weight
        return F.normalize(w.float(), dim=-1).to(w.dtype) if self.arch.norm_head else w

    def hidden_states(self, input_ids, meta, caches=None, inputs_embeds=None):
        x = inputs_embeds if inputs_embeds is not None else self.model.embed_tokens(input_ids.reshape(-1))
        x = x.reshape(-1, x.shape[-1])
        delta, residual = x, None
        for i, layer in enumerate(self.model.layers):
            cache = caches[i] if caches is not None else None
            if self.gradient_checkpointing and self.training and cache is None:
                from torch.utils.checkpoint import checkpoint
                delta, residual = checkpoint(lambda d, r, _l=layer: _l(d, r, meta), delta, residual, use_reentrant=False)
            else:
                delta, residual = layer(delta, residual, meta, cache)
        if residual is None:
            return self.model.norm(delta)
        return self.model.norm(delta, residual)[0]

    def forward(self, input_ids=None, attention_mask=None, labels=None, position_ids=None, cu_seqlens=None,
                inputs_embeds=None, return_dict=True, **_):
        b, s = input_ids.shape
        dev = self.lm_head.weight.device
        # a batch handed over on the host is parsed there and copied (no read-back from the GPU per micro-batch)
        meta = build_meta(input_ids, attention_mask, position_ids, cu_seqlens, device=dev)
        input_ids = input_ids.to(dev, non_blocking=True)
        if labels is not None:
            labels = labels.to(dev, non_blocking=True)
        h = self.hidden_states(input_ids, meta, inputs_embeds=inputs_embeds)
        out = {}
        if labels is not None:
            # HF convention: the model shifts — position t predicts labels[t + 1]
            shift = torch.full_like(labels, -100)
            shift[:, :-1] = labels[:, 1:]
            flat = shift.reshape(-1)
            valid = flat != -100
            tok = ops.lm_head_cross_entropy(h, self.head_weight(), flat.masked_fill(~valid, 0))
            out["loss"] = (tok * valid).sum() / valid.sum().clamp(min=1)
            with torch.no_grad():
                out["num_tokens"] = valid.sum()
        else:
            out["logits"] = ops.linear(h, self.head_weight()).view(b, s, -1)
        return out

    # ---- generation -----------------------------------------------------------------------------
    @torch.no_grad()
    def _decode_steps(self, input_ids, max_new_tokens=64, do_sample=False, temperature=1.0, top_k=0, top_p=0.0,
                      eos_token_id=None, repetition_penalty=1.0, stop_words_ids=None, soft_prefix=None, **_):
        """Greedy / sampled decoding with per-layer KV caches; yields the running ``[b, s]`` token tensor after
        every new token.  A row ends at ``eos_token_id`` or when its tail equals one of ``stop_words_ids`` (token
        sequences; the stop sequence stays in the output, later positions are filled with eos).
        ``soft_prefix``: ``{"embeds": [P, hidden]}`` (prompt tuning: virtual input embeddings in front of the
        prompt) or ``{"kv": [layers, 2, P, kv_heads, head_dim]}`` (prefix tuning: pre-filled cache entries)."""
        from ...infer.generation import sample_next
        a = self.arch
        eos = a.eos_token_id if eos_token_id is None else eos_token_id
        stops = [torch.tensor(w, dtype=torch.long, device=input_ids.device) for w in (stop_words_ids or []) if len(w)]
        b, s = input_ids.shape
        dev, dt = input_ids.device, self.lm_head.weight.dtype
        soft = soft_prefix or {}
        pre_kv = soft.get("kv")
        pre_emb = soft.get("embeds")
        n_kv = 0 if pre_kv is None else pre_kv.shape[2]
        n_emb = 0 if pre_emb is None else pre_emb.shape[0]
        room = s + max_new_tokens + n_kv + n_emb
        if a.use_cache_quantization:
            from .kv_quant import QuantizedKV
            caches = [{"kq": QuantizedKV(b, room, a.kv_heads, a.head_dim, dev, dt),
                       "vq": QuantizedKV(b, room, a.kv_heads, a.head_dim, dev, dt), "len": 0}
                      for _ in range(a.num_hidden_layers)]
        else:
            caches = [{"k": torch.zeros(b, room, a.kv_heads, a.head_dim, dtype=dt, device=dev),
                       "v": torch.zeros(b, room, a.kv_heads, a.head_dim, dtype=dt, device=dev), "len": 0}
                      for _ in range(a.num_hidden_layers)]
        if n_kv:
            for l, c in enumerate(caches):
                k0, v0 = (pre_kv[l, i].to(dt).unsqueeze(0).expand(b, -1, -1, -1) for i in (0, 1))
                if "kq" in c:
                    c["kq"].append(0, k0); c["vq"].append(0, v0)
                else:
                    c["k"][:, :n_kv], c["v"][:, :n_kv] = k0, v0
                c["len"] = n_kv
        toks = input_ids
        done = torch.zeros(b, dtype=torch.bool, device=dev)
        fill = eos if eos is not None else 0
        for step in range(max_new_tokens):
            inp = toks if step == 0 else toks[:, -1:]
            p0 = n_kv if step == 0 else n_kv + n_emb + toks.shape[1] - 1
            embeds = None
            if step == 0 and n_emb:
                embeds = torch.cat((pre_emb.to(dt).unsqueeze(0).expand(b, -1, -1), self.model.embed_tokens(inp)), 1)
                inp = torch.cat((inp.new_zeros(b, n_emb), inp), 1)          # shapes only: the embeddings are given
            pos = torch.arange(inp.shape[1], device=dev).unsqueeze(0).expand(b, -1) + p0
            meta = build_meta(inp, None, pos)
            h = self.hidden_states(inp, meta, caches, inputs_embeds=embeds)
            logits = ops.linear(h.view(b, inp.shape[1], -1)[:, -1], self.head_weight()).float()
            if repetition_penalty != 1.0:
                seen = torch.gather(logits, 1, toks)
                logits.scatter_(1, toks, torch.where(seen > 0, seen / repetition_penalty, seen * repetition_penalty))
            nxt = sample_next(logits, temperature, top_k, top_p, greedy=not do_sample)
            if eos is not None or stops:
                nxt = torch.where(done, torch.full_like(nxt, fill), nxt)
            toks = torch.cat((toks, nxt.unsqueeze(1)), 1)
            if eos is not None:
                done |= nxt == eos
            new_len = toks.shape[1] - s
            for w in stops:
                if new_len >= len(w):
                    done |= (toks[:, -len(w):] == w).all(dim=1)
            yield toks
            if (eos is not None or stops) and bool(done.all()):
                break

    def generate(self, input_ids, attention_mask=None, max_new_tokens=64, num_beams=1, **kw):
        toks = input_ids
        for toks in self._decode_steps(input_ids, max_new_tokens=max_new_tokens, **kw):
            pass
        return toks

    def generate_stream(self, input_ids, max_new_tokens=64, **kw):
        """Yields the newest token of every row (``[b]``) as soon as it is decoded."""
        for toks in self._decode_steps(input_ids, max_new_tokens=max_new_tokens, **kw):
            yield toks[:, -1]

    # ---- checkpoint IO --------------------------------------------------------------------------------
    def canonical_state(self):
        return {k: v for k, v in self.state_dict().items()}

    def save_pretrained(self, path, state_dict=None, family_format=True, safe_serialization=False, **_):
        from .io import export_state
        os.makedirs(path, exist_ok=True)
        sd = state_dict if state_dict is not None else self.state_dict()
        sd = export_state({k: v.detach().cpu() for k, v in sd.items()}, self.arch) if family_format else sd
        torch.save(sd, os.path.join(path, "pytorch_model.bin"))
        from .io import export_config
        with open(os.path.join(path, "config.json"), "w") as f:
            json.dump(export_config(self.arch), f, indent=2)

    @classmethod
    def from_pretrained(cls, path, family=None, torch_dtype=torch.float32, arch_overrides=None, **_):
        from .io import import_state
        with open(os.path.join(path, "config.json")) as f:
            cfg = json.load(f)
        arch = arch_from_hf_config(cfg, family)
        for k, v in (arch_overrides or {}).items():
            setattr(arch, k, v)
        if isinstance(torch_dtype, str):
            torch_dtype = getattr(torch, torch_dtype.replace("torch.", ""))
        model = cls(arch, torch_dtype)
        from ...ckpt.hf_import import load_hf_state
        sd = import_state(load_hf_state(path), arch)
        missing, unexpected = model.load_state_dict({k: v.to(torch_dtype) for k, v in sd.items()}, strict=False)
        missing = [m for m in missing if not (arch.tie_word_embeddings and m == "lm_head.weight")]
        if missing or unexpected:
            raise RuntimeError(f"from_pretrained({path}): missing {missing[:8]}, unexpected {unexpected[:8]}")
        if arch.tie_word_embeddings:
            model.lm_head.weight = model.model.embed_tokens.weight
        return model
