"""Qwen-VL: the Qwen decoder + a ViT image tower and a cross-attention resampler.

Parity: llm/models/hf_models/qwen_vl/visual.py:93-425 and modeling_qwen.py:113-703 — images referenced in the
prompt between the ``<img>`` / ``</img>`` tokens are encoded by a ViT (patch conv → pre-LN transformer), compressed
to ``n_queries`` tokens by one cross-attention layer with learned queries and 2-D sin-cos position embeddings,
normalised, projected to the LM width and written over the image-pad token positions of the input embeddings.

The tower's parameters carry the names of the released checkpoint (``conv1``, ``positional_embedding``, ``ln_pre``,
``transformer.resblocks.N.{ln_1, ln_2, attn.in_proj, attn.out_proj, mlp.c_fc, mlp.c_proj}``,
``attn_pool.{pos_embed, query, kv_proj, attn.in_proj_weight, ..., ln_q, ln_kv}``, ``ln_post``, ``proj``), so a
checkpoint's ``transformer.visual.*`` tensors load with ``load_state_dict`` unchanged; ``from_pretrained`` /
``save_pretrained`` read and write the HF folder layout (decoder names through the Qwen name map of ``io.py``).
The tower runs on PyTorch library attention: it sees each image once per sample and is not a training hot path.
"""
from __future__ import annotations

import json
import math
import os
from collections import OrderedDict
from typing import List, Optional

import numpy as np
import torch
import torch.nn as nn
import torch.nn.functional as F

from ...config.registry import MODULE_ZOO_REGISTRY
from .modeling import CausalLM, HFArch

IMAGE_MEAN = (0.48145466, 0.4578275, 0.40821073)
IMAGE_STD = (0.26862954, 0.26130258, 0.27577711)


def sincos_2d(dim, grid):
    """2-D sin-cos table ``[grid², dim]``: the first half of the channels encodes the column, the second the row
    (visual.py:42-88, the MAE construction with "w goes first")."""
    def one(d, pos):
        omega = 1.0 / 10000 ** (np.arange(d // 2, dtype=np.float32) / (d / 2.0))
        out = np.einsum("m,d->md", pos.reshape(-1), omega)
        return np.concatenate([np.sin(out), np.cos(out)], axis=1)
    gw, gh = np.meshgrid(np.arange(grid, dtype=np.float32), np.arange(grid, dtype=np.float32))
    return torch.from_numpy(np.concatenate([one(dim // 2, gw), one(dim // 2, gh)], axis=1)).float()


def abs_pos_for(table, n_tokens):
    """Bicubic resize of a square position table ``[s², C]`` to ``n_tokens`` positions (visual.py:21-39)."""
    src, tgt = int(math.sqrt(table.shape[0])), int(math.sqrt(n_tokens))
    if src == tgt:
        return table
    t = F.interpolate(table.float().reshape(1, src, src, -1).permute(0, 3, 1, 2), size=(tgt, tgt), mode="bicubic",
                      align_corners=False)
    return t.permute(0, 2, 3, 1).flatten(0, 2).to(table.dtype)


class Resampler(nn.Module):
    """``grid_size²`` learned queries cross-attend over the patch tokens (visual.py:93-154)."""

    def __init__(self, grid_size, embed_dim, num_heads, kv_dim=None):
        super().__init__()
        self.num_queries = grid_size ** 2
        self.embed_dim, self.num_heads = embed_dim, num_heads
        self.pos_embed = nn.Parameter(sincos_2d(embed_dim, grid_size), requires_grad=False)
        self.query = nn.Parameter(torch.zeros(self.num_queries, embed_dim))
        nn.init.trunc_normal_(self.query, std=0.02)
        self.kv_proj = (nn.Linear(kv_dim, embed_dim, bias=False) if kv_dim is not None and kv_dim != embed_dim
                        else nn.Identity())
        self.attn = nn.MultiheadAttention(embed_dim, num_heads)          # sequence-first, as in the checkpoint
        self.ln_q = nn.LayerNorm(embed_dim, eps=1e-6)
        self.ln_kv = nn.LayerNorm(embed_dim, eps=1e-6)

    def forward(self, x):                                               # x [B, L, kv_dim]
        pos_k = abs_pos_for(self.pos_embed, x.shape[1])
        kv = self.ln_kv(self.kv_proj(x)).permute(1, 0, 2)               # [L, B, C]
        q = self.ln_q(self.query).unsqueeze(1).expand(-1, x.shape[0], -1)
        out = self.attn(q + self.pos_embed.unsqueeze(1).to(q.dtype), kv + pos_k.unsqueeze(1).to(kv.dtype), kv,
                        need_weights=False)[0]
        return out.permute(1, 0, 2)                                     # [B, Q, C]


class VisualAttention(nn.Module):
    """Self-attention whose fused ``in_proj`` packs (q, k, v) per head: output channel
    ``head · 3d + {0, d, 2d} + i`` (visual.py:182-200)."""

    def __init__(self, embed_dim, num_heads):
        super().__init__()
        self.num_heads, self.head_dim = num_heads, embed_dim // num_heads
        self.in_proj = nn.Linear(embed_dim, 3 * embed_dim)
        self.out_proj = nn.Linear(embed_dim, embed_dim)

    def forward(self, x):                                               # [B, L, C]
        B, L, C = x.shape
        qkv = self.in_proj(x).view(B, L, self.num_heads, 3 * self.head_dim)
        q, k, v = (t.transpose(1, 2) for t in qkv.split(self.head_dim, dim=-1))   # [B, H, L, d]
        o = F.scaled_dot_product_attention(q, k, v)
        return self.out_proj(o.transpose(1, 2).reshape(B, L, C))


class VisualAttentionBlock(nn.Module):
    def __init__(self, d_model, n_head, mlp_ratio=4.0):
        super().__init__()
        self.ln_1 = nn.LayerNorm(d_model, eps=1e-6)
        self.ln_2 = nn.LayerNorm(d_model, eps=1e-6)
        self.attn = VisualAttention(d_model, n_head)
        width = int(d_model * mlp_ratio)
        self.mlp = nn.Sequential(OrderedDict([("c_fc", nn.Linear(d_model, width)), ("gelu", nn.GELU()),
                                              ("c_proj", nn.Linear(width, d_model))]))

    def forward(self, x):
        x = x + self.attn(self.ln_1(x))
        return x + self.mlp(self.ln_2(x))


class TransformerBlock(nn.Module):
    def __init__(self, width, layers, heads, mlp_ratio=4.0):
        super().__init__()
        self.resblocks = nn.ModuleList(VisualAttentionBlock(width, heads, mlp_ratio) for _ in range(layers))

    def forward(self, x):
        for blk in self.resblocks:
            x = blk(x)
        return x


class VisionTransformer(nn.Module):
    """ViT-bigG tower of Qwen-VL (visual.py:331-405).  The position table always covers a 16 x 16 grid and is resized
    to the image's patch grid."""

    def __init__(self, image_size=448, patch_size=14, width=1664, layers=48, heads=16, mlp_ratio=4.9231,
                 n_queries=256, output_dim=4096, **_ignored):
        super().__init__()
        self.image_size, self.patch_size, self.output_dim = image_size, patch_size, output_dim
        self.conv1 = nn.Conv2d(3, width, patch_size, patch_size, bias=False)
        self.positional_embedding = nn.Parameter(width ** -0.5 * torch.randn(256, width))
        self.ln_pre = nn.LayerNorm(width, eps=1e-6)
        self.transformer = TransformerBlock(width, layers, heads, mlp_ratio)
        self.attn_pool = Resampler(int(math.sqrt(n_queries)), output_dim, output_dim // 128, kv_dim=width)
        self.ln_post = nn.LayerNorm(output_dim, eps=1e-6)
        self.proj = nn.Parameter(output_dim ** -0.5 * torch.randn(output_dim, output_dim))

    def forward(self, images):                                          # [N, 3, S, S] → [N, n_queries, output_dim]
        x = self.conv1(images.to(self.conv1.weight.dtype)).flatten(2).transpose(1, 2)
        x = self.ln_pre(x + abs_pos_for(self.positional_embedding, x.shape[1]).to(x.dtype))
        x = self.transformer(x)
        x = self.ln_post(self.attn_pool(x))
        return x @ self.proj

    def preprocess(self, image):
        """PIL image → normalised ``[3, S, S]`` tensor (bicubic resize, CLIP mean / std; visual.py:353-360)."""
        from PIL import Image
        img = image.convert("RGB").resize((self.image_size, self.image_size), Image.BICUBIC)
        t = torch.from_numpy(np.asarray(img, dtype=np.float32) / 255.0).permute(2, 0, 1)
        mean, std = torch.tensor(IMAGE_MEAN).view(3, 1, 1), torch.tensor(IMAGE_STD).view(3, 1, 1)
        return (t - mean) / std

    def encode(self, image_paths: List[str]):
        """Local image files → features (visual.py:407-425; remote URLs need a network and are refused here)."""
        from PIL import Image
        ims = []
        for path in image_paths:
            if path.startswith(("http://", "https://")):
                raise ValueError(f"remote image {path!r}: download it first, this process has no network access")
            ims.append(self.preprocess(Image.open(path)))
        dev = self.conv1.weight.device
        return self(torch.stack(ims).to(dev))


class QWenVL(CausalLM):
    """Qwen decoder whose image-pad positions are overwritten by the tower's features.

    An image is announced in the token stream as ``<img>`` + pad tokens + ``</img>`` (ids ``image_start_id``,
    ``image_start_id + 2`` and ``image_start_id + 1``; the tokenizer writes the UTF-8 bytes of the image path into
    the first pad positions, modeling_qwen.py:332-343).  ``images`` (pre-processed pixels ``[N, 3, S, S]``, in order of
    appearance) may be passed instead of letting the model open the files."""

    def __init__(self, arch: HFArch, dtype=torch.float32, visual_cfg=None, image_start_id=151857):
        super().__init__(arch, dtype)
        v = dict(visual_cfg or {})
        self.image_start_id = int(v.pop("image_start_id", image_start_id))
        v.setdefault("output_dim", arch.hidden_size)
        self.visual_cfg = dict(v, image_start_id=self.image_start_id)
        self.visual = VisionTransformer(**v).to(dtype)

    def image_paths(self, input_ids):
        """Paths written into the pad positions between each ``<img>`` / ``</img>`` pair."""
        ids = input_ids.tolist()
        out = []
        for row in ids:
            i = 0
            while i < len(row):
                if row[i] == self.image_start_id:
                    j = row.index(self.image_start_id + 1, i)
                    body = row[i + 1:j]
                    if self.image_start_id + 2 in body:
                        body = body[:body.index(self.image_start_id + 2)]
                    out.append(bytes(body).decode("utf-8"))
                    i = j
                i += 1
        return out

    def embed_with_images(self, input_ids, images=None):
        """Token embeddings with every image's features written between its ``<img>`` and ``</img>`` tokens."""
        emb = self.model.embed_tokens(input_ids)
        starts = torch.nonzero(input_ids == self.image_start_id)
        if starts.numel() == 0:
            return emb
        ends = torch.nonzero(input_ids == self.image_start_id + 1)
        if starts.shape[0] != ends.shape[0]:
            raise ValueError("unbalanced <img> / </img> tokens")
        feats = self.visual(images) if images is not None else self.visual.encode(self.image_paths(input_ids))
        if feats.shape[0] != starts.shape[0]:
            raise ValueError(f"{starts.shape[0]} image spans in the prompt but {feats.shape[0]} images")
        emb = emb.clone()
        for n, ((b, s), (b2, e)) in enumerate(zip(starts.tolist(), ends.tolist())):
            if b != b2 or e - s - 1 != feats.shape[1]:
                raise ValueError(f"image span {n} holds {e - s - 1} pad tokens, the tower emits {feats.shape[1]}")
            emb[b, s + 1:e] = feats[n].to(emb.dtype)
        return emb

    def forward(self, input_ids=None, images=None, **kw):
        if images is not None or bool((input_ids == self.image_start_id).any()):
            dev = self.lm_head.weight.device
            kw["inputs_embeds"] = self.embed_with_images(input_ids.to(dev), None if images is None else images.to(dev))
        return super().forward(input_ids=input_ids, **kw)

    # ---- HF folder layout -------------------------------------------------------------------------------------
    def save_pretrained(self, path):
        """``config.json`` (decoder fields + the ``visual`` block) and one ``pytorch_model.bin`` with the decoder under
        its Qwen names and the tower under ``transformer.visual.``."""
        from .io import export_config, export_state
        os.makedirs(path, exist_ok=True)
        sd = {k: v.detach().cpu() for k, v in self.state_dict().items()}
        lm = export_state({k: v for k, v in sd.items() if not k.startswith("visual.")}, self.arch)
        lm.update({"transformer." + k: v for k, v in sd.items() if k.startswith("visual.")})
        torch.save(lm, os.path.join(path, "pytorch_model.bin"))
        cfg = export_config(self.arch)
        cfg.update(architectures=["QWenLMHeadModel"], visual=self.visual_cfg)
        with open(os.path.join(path, "config.json"), "w") as f:
            json.dump(cfg, f, indent=1, default=str)

    @classmethod
    def from_pretrained(cls, path, dtype=torch.bfloat16, arch: Optional[HFArch] = None, **_):
        """Load a Qwen-VL folder (``config.json`` with a ``visual`` block + ``.bin`` / ``.safetensors`` shards)."""
        from ...ckpt.hf_import import load_hf_state
        from .io import import_state
        from .modeling import arch_from_hf_config
        with open(os.path.join(path, "config.json")) as f:
            cfg = json.load(f)
        arch = arch or arch_from_hf_config(cfg, "qwen")
        model = cls(arch, dtype, cfg.get("visual"))
        raw = load_hf_state(path)
        tower = {k[len("transformer."):]: v for k, v in raw.items() if k.startswith("transformer.visual.")}
        lm = import_state({k: v for k, v in raw.items() if not k.startswith("transformer.visual.")}, arch)
        missing, unexpected = model.load_state_dict({k: v.to(dtype) for k, v in {**lm, **tower}.items()}, strict=False)
        missing = [m for m in missing if "rotary" not in m and "inv_freq" not in m]
        if missing or unexpected:
            raise ValueError(f"Qwen-VL checkpoint does not match the model: missing {missing[:5]}, "
                             f"unexpected {list(unexpected)[:5]}")
        return model.to(dtype)


@MODULE_ZOO_REGISTRY.register("QWenForVL")
def build_qwen_vl(**cfg):
    from . import get_model_cfg
    mc = get_model_cfg(cfg)
    if cfg.get("arch") is not None:
        return QWenVL(HFArch(family="qwen", **cfg["arch"]), mc["torch_dtype"], cfg.get("visual"))
    path = cfg.get("model_name_or_path") or cfg.get("pretrained_model_name_or_path")
    if not path:
        raise ValueError("QWenForVL needs `arch` (+ `visual`) to build from scratch or `model_name_or_path` to load")
    return QWenVL.from_pretrained(path, mc["torch_dtype"])
