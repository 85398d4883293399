"""Qwen-VL: the Qwen decoder + a ViT image tower and a cross-attention resampler.

Parity: llm/models/hf_models/qwen_vl/visual.py:93-425 and modeling_qwen.py:113-703 — images
referenced in the prompt between ``<img>`` … ``</img>`` tokens are encoded by a ViT
(patch conv → pre-LN transformer → post-LN), compressed to ``n_queries`` tokens by one
cross-attention layer with learned queries and 2-D sin-cos position embeddings, projected to
the LM width and written over the image-pad token positions of the input embeddings.
"""
from __future__ import annotations

import math

import numpy as np
import torch
import torch.nn as nn
import torch.nn.functional as F

from ...config.registry import MODULE_ZOO_REGISTRY
from .modeling import CausalLM, HFArch


def sincos_2d(dim, grid):
    def one(d, pos):
        omega = 1.0 / 10000 ** (np.arange(d // 2, dtype=np.float64) / (d / 2.0))
        out = np.einsum("m,d->md", pos.reshape(-1), omega)
        return np.concatenate([np.sin(out), np.cos(out)], axis=1)
    gh, gw = np.meshgrid(np.arange(grid, dtype=np.float32), np.arange(grid, dtype=np.float32), indexing="ij")
    return torch.from_numpy(np.concatenate([one(dim // 2, gw), one(dim // 2, gh)], axis=1)).float()


class Resampler(nn.Module):
    def __init__(self, grid_size, embed_dim, num_heads, kv_dim):
        super().__init__()
        self.num_queries = grid_size ** 2
        self.pos_embed = nn.Parameter(sincos_2d(embed_dim, grid_size), requires_grad=False)
        self.query = nn.Parameter(torch.zeros(self.num_queries, embed_dim))
        nn.init.trunc_normal_(self.query, std=0.02)
        self.kv_proj = nn.Linear(kv_dim, embed_dim, bias=False) if kv_dim != embed_dim else nn.Identity()
        self.attn = nn.MultiheadAttention(embed_dim, num_heads, batch_first=True)
        self.ln_q, self.ln_kv = nn.LayerNorm(embed_dim, eps=1e-6), nn.LayerNorm(embed_dim, eps=1e-6)

    def forward(self, x):
        n = x.shape[1]
        g = int(math.sqrt(n))
        pos_k = self.pos_embed
        if n != self.num_queries:       # interpolate key positions to the patch grid
            src = int(math.sqrt(self.num_queries))
            pos_k = F.interpolate(self.pos_embed.view(1, src, src, -1).permute(0, 3, 1, 2), size=(g, g), mode="bicubic",
                                  align_corners=False).permute(0, 2, 3, 1).reshape(n, -1)
        kv = self.ln_kv(self.kv_proj(x))
        q = self.ln_q(self.query).unsqueeze(0).expand(x.shape[0], -1, -1)
        out, _ = self.attn(q + self.pos_embed.unsqueeze(0), kv + pos_k.unsqueeze(0).to(kv.dtype), kv)
        return out


class VisionTransformer(nn.Module):
    def __init__(self, image_size=448, patch_size=14, width=1664, layers=48, heads=16, mlp_ratio=4.9231,
                 n_queries=256, output_dim=4096):
        super().__init__()
        self.grid = image_size // patch_size
        self.conv1 = nn.Conv2d(3, width, patch_size, patch_size, bias=False)
        self.positional_embedding = nn.Parameter(width ** -0.5 * torch.randn(self.grid ** 2, width))
        self.ln_pre, self.ln_post = nn.LayerNorm(width, eps=1e-6), nn.LayerNorm(output_dim, eps=1e-6)
        layer = nn.TransformerEncoderLayer(width, heads, int(width * mlp_ratio), dropout=0.0, activation="gelu",
                                           batch_first=True, norm_first=True)
        self.transformer = nn.TransformerEncoder(layer, layers)
        self.attn_pool = Resampler(int(math.sqrt(n_queries)), output_dim, output_dim // 128, width)
        self.proj = nn.Parameter(output_dim ** -0.5 * torch.randn(output_dim, output_dim))

    def forward(self, images):
        x = self.conv1(images).flatten(2).transpose(1, 2)
        x = self.ln_pre(x + self.positional_embedding.to(x.dtype))
        x = self.transformer(x)
        x = self.ln_post(self.attn_pool(x))
        return x @ self.proj


class QWenVL(CausalLM):
    def __init__(self, arch: HFArch, dtype=torch.float32, visual_cfg=None, image_start_id=151857):
        super().__init__(arch, dtype)
        v = dict(visual_cfg or {})
        v.setdefault("output_dim", arch.hidden_size)
        self.visual = VisionTransformer(**v).to(dtype)
        self.image_start_id = image_start_id

    def forward(self, input_ids=None, images=None, **kw):
        if images is not None:
            emb = self.model.embed_tokens(input_ids)
            feats = self.visual(images.to(emb.dtype))
            starts = torch.nonzero(input_ids == self.image_start_id)
            for n, (b, s) in enumerate(starts.tolist()):
                emb[b, s + 1:s + 1 + feats.shape[1]] = feats[n]
            kw["inputs_embeds"] = emb
        return super().forward(input_ids=input_ids, **kw)


@MODULE_ZOO_REGISTRY.register("QWenForVL")
def build_qwen_vl(**cfg):
    from . import get_model_cfg
    mc = get_model_cfg(cfg)
    if cfg.get("arch") is not None:
        return QWenVL(HFArch(family="qwen", **cfg["arch"]), mc["torch_dtype"], cfg.get("visual"))
    raise NotImplementedError("loading Qwen-VL checkpoints needs the tower weights; build from `arch`/`visual` "
                              "and load_state_dict explicitly")
