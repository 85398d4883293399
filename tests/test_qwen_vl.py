"""Qwen-VL (H9): the image tower's parameter names are the released checkpoint's, a tiny random model survives
``save_pretrained`` → ``from_pretrained`` in the HF folder layout, and image features land exactly on the pad
positions between ``<img>`` and ``</img>``.  Names checked against
llm/models/hf_models/qwen_vl/visual.py:93-425 of the reference."""
import json
import os

import pytest
import torch

from easyllm_b200.models.hf_models.modeling import HFArch
from easyllm_b200.models.hf_models.qwen_vl import QWenVL, VisionTransformer, abs_pos_for, sincos_2d

IMG_START = 900


def _tiny():
    arch = HFArch(family="qwen", vocab_size=1024, hidden_size=128, intermediate_size=256, num_hidden_layers=2,
                  num_attention_heads=2, num_key_value_heads=2, max_position_embeddings=128, qkv_bias=True)
    visual = dict(image_size=56, patch_size=14, width=64, layers=2, heads=2, mlp_ratio=2.0, n_queries=4,
                  image_start_id=IMG_START)
    torch.manual_seed(0)
    return QWenVL(arch, torch.float32, visual)


def test_tower_parameter_names_match_the_released_checkpoint():
    v = VisionTransformer(image_size=56, patch_size=14, width=64, layers=2, heads=2, mlp_ratio=2.0, n_queries=4,
                          output_dim=128)
    names = set(v.state_dict())
    want = {"conv1.weight", "positional_embedding", "ln_pre.weight", "ln_pre.bias", "ln_post.weight", "ln_post.bias",
            "proj", "attn_pool.pos_embed", "attn_pool.query", "attn_pool.kv_proj.weight",
            "attn_pool.attn.in_proj_weight", "attn_pool.attn.in_proj_bias", "attn_pool.attn.out_proj.weight",
            "attn_pool.attn.out_proj.bias", "attn_pool.ln_q.weight", "attn_pool.ln_q.bias", "attn_pool.ln_kv.weight",
            "attn_pool.ln_kv.bias"}
    for i in range(2):
        for leaf in ("ln_1.weight", "ln_1.bias", "ln_2.weight", "ln_2.bias", "attn.in_proj.weight", "attn.in_proj.bias",
                     "attn.out_proj.weight", "attn.out_proj.bias", "mlp.c_fc.weight", "mlp.c_fc.bias",
                     "mlp.c_proj.weight", "mlp.c_proj.bias"):
            want.add(f"transformer.resblocks.{i}.{leaf}")
    assert names == want
    assert v.state_dict()["positional_embedding"].shape == (256, 64)          # always a 16 x 16 table
    assert v.state_dict()["attn_pool.attn.in_proj_weight"].shape == (3 * 128, 128)


def test_tower_attention_uses_the_per_head_qkv_packing():
    """``in_proj`` packs (q, k, v) per head; against an explicit restatement of that layout."""
    from easyllm_b200.models.hf_models.qwen_vl import VisualAttention
    torch.manual_seed(1)
    a = VisualAttention(32, 4)
    x = torch.randn(2, 5, 32)
    qkv = a.in_proj(x).view(2, 5, 4, 24)
    q, k, v = qkv[..., :8], qkv[..., 8:16], qkv[..., 16:]
    s = torch.einsum("blhd,bmhd->bhlm", q, k) / 8 ** 0.5
    o = torch.einsum("bhlm,bmhd->blhd", s.softmax(-1), v).reshape(2, 5, 32)
    torch.testing.assert_close(a(x), a.out_proj(o), rtol=1e-5, atol=1e-5)


def test_position_tables():
    t = sincos_2d(8, 2)                  # first half of the channels: column, second half: row
    assert t.shape == (4, 8) and torch.allclose(t[0], t[0]) and not torch.allclose(t[0, :4], t[1, :4])
    assert torch.allclose(t[0, 4:], t[1, 4:])                   # same row, different column
    big = abs_pos_for(torch.randn(16, 6), 64)
    assert big.shape == (64, 6)


def test_image_features_replace_exactly_the_pad_span(tmp_path):
    m = _tiny().eval()
    n_q = 4
    ids = torch.randint(0, 800, (2, 24))
    for b, s in ((0, 3), (1, 10)):
        ids[b, s] = IMG_START
        ids[b, s + 1:s + 1 + n_q] = IMG_START + 2
        ids[b, s + 1 + n_q] = IMG_START + 1
    images = torch.randn(2, 3, 56, 56)
    with torch.no_grad():
        emb = m.embed_with_images(ids, images)
        feats = m.visual(images)
        plain = m.model.embed_tokens(ids)
    for n, (b, s) in enumerate(((0, 3), (1, 10))):
        torch.testing.assert_close(emb[b, s + 1:s + 1 + n_q], feats[n])
        mask = torch.ones(24, dtype=torch.bool)
        mask[s + 1:s + 1 + n_q] = False
        torch.testing.assert_close(emb[b][mask], plain[b][mask])        # every other position is untouched
    out = m(input_ids=ids, images=images, labels=ids)
    assert torch.isfinite(out["loss"])
    out["loss"].backward()
    assert m.visual.conv1.weight.grad is not None and m.visual.conv1.weight.grad.abs().sum() > 0
    bad = ids.clone()
    bad[0, 3 + 1 + n_q] = 5                                             # a missing </img>
    with pytest.raises(ValueError):
        m.embed_with_images(bad, images)


def test_image_paths_are_read_from_the_pad_tokens_and_files_are_encoded(tmp_path):
    from PIL import Image
    m = _tiny().eval()
    path = str(tmp_path / "a.png")
    Image.fromarray((torch.rand(40, 30, 3) * 255).to(torch.uint8).numpy()).save(path)
    body = list(path.encode("utf-8"))
    n_pad = 4
    assert len(body) > n_pad                      # real prompts reserve 256 pads; the tiny tower emits 4 features
    m.visual.attn_pool.num_queries  # noqa: B018
    ids = torch.full((1, len(body) + 8), 7)
    ids[0, 1] = IMG_START
    ids[0, 2:2 + len(body)] = torch.tensor(body)
    ids[0, 2 + len(body)] = IMG_START + 1
    assert m.image_paths(ids) == [path]
    with torch.no_grad():
        f = m.visual.encode([path])
    assert f.shape == (1, 4, 128)
    with pytest.raises(ValueError, match="network"):
        m.visual.encode(["https://example.com/x.png"])


def test_save_and_from_pretrained_round_trip(tmp_path):
    m = _tiny().eval()
    d = str(tmp_path / "qwen_vl")
    m.save_pretrained(d)
    keys = set(torch.load(os.path.join(d, "pytorch_model.bin")))
    assert "transformer.visual.conv1.weight" in keys and "transformer.visual.attn_pool.attn.in_proj_weight" in keys
    assert "transformer.h.0.attn.c_attn.weight" in keys and "transformer.wte.weight" in keys
    with open(os.path.join(d, "config.json")) as f:
        cfg = json.load(f)
    assert cfg["visual"]["image_start_id"] == IMG_START and cfg["model_type"] == "qwen"
    m2 = QWenVL.from_pretrained(d, torch.float32).eval()
    sd1, sd2 = m.state_dict(), m2.state_dict()
    assert set(sd1) == set(sd2)
    for k in sd1:
        torch.testing.assert_close(sd1[k], sd2[k], msg=k)
    ids = torch.randint(0, 800, (1, 16))
    ids[0, 2] = IMG_START; ids[0, 3:7] = IMG_START + 2; ids[0, 7] = IMG_START + 1
    images = torch.randn(1, 3, 56, 56)
    with torch.no_grad():
        a = m(input_ids=ids, images=images)["logits"]
        b = m2(input_ids=ids, images=images)["logits"]
    torch.testing.assert_close(a, b)
    # the registry entry loads the same folder
    from easyllm_b200.config.registry import MODULE_ZOO_REGISTRY
    m3 = MODULE_ZOO_REGISTRY.build({"type": "QWenForVL", "kwargs": {"model_name_or_path": d, "torch_dtype": "float32"}})
    torch.testing.assert_close(m3.state_dict()["visual.proj"], sd1["visual.proj"])
