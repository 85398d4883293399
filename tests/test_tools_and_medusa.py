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


def test_convert_colossalai_shards_to_hf(tmp_path):
    """pp=2 x tp=2 ColossalAI-style shards (stage-local layer numbers, interleaved rotary layout) round-trip to HF."""
    tool = _tool("convert_colossalai_hf")
    torch.manual_seed(1)
    h, ffn, heads, vocab, layers = 32, 48, 4, 40, 2
    hf = {"model.embed_tokens.weight": torch.randn(vocab, h), "model.norm.weight": torch.randn(h),
          "lm_head.weight": torch.randn(vocab, h)}
    for li in range(layers):
        p = f"model.layers.{li}."
        for n, shape in (("self_attn.q_proj", (h, h)), ("self_attn.k_proj", (h, h)), ("self_attn.v_proj", (h, h)),
                         ("self_attn.o_proj", (h, h)), ("mlp.gate_proj", (ffn, h)), ("mlp.up_proj", (ffn, h)),
                         ("mlp.down_proj", (h, ffn))):
            hf[p + n + ".weight"] = torch.randn(*shape)
        hf[p + "input_layernorm.weight"] = torch.randn(h)
        hf[p + "post_attention_layernorm.weight"] = torch.randn(h)

    def interleave(w):            # HF half-rotation layout -> interleaved pairs (the source layout)
        return w.view(heads, 2, h // heads // 2, h).transpose(1, 2).reshape(h, h)

    back = {v: k for k, v in tool.NAME.items()}
    src = tmp_path / "shards"
    os.makedirs(src)
    for pp in range(2):               # one layer per stage, numbered from 0 inside the stage
        full = {}
        for n, sub in back.items():
            w = hf[f"model.layers.{pp}.{n}.weight"]
            if n in ("self_attn.q_proj", "self_attn.k_proj"):
                w = interleave(w)
            full[f"model.layers.0.{sub}.weight"] = w
        if pp == 0:
            full["model.tok_embeddings.weight"] = hf["model.embed_tokens.weight"]
        else:
            full["model.norm.weight"] = hf["model.norm.weight"]
            full["model.output.weight"] = hf["lm_head.weight"]
        for tp in range(2):
            shard = {}
            for k, w in full.items():
                if any(c in k for c in tool.COL):
                    shard[k] = w.chunk(2, 0)[tp].clone()
                elif any(c in k for c in tool.ROW):
                    shard[k] = w.chunk(2, 1)[tp].clone()
                else:
                    shard[k] = w.clone()
            torch.save(shard, src / f"model_tp{tp}_pp{pp}.pt")
    out = tmp_path / "hf"
    tool.main(["--input_dir", str(src), "--output_dir", str(out), "--n_heads", str(heads), "--dim", str(h)])
    got = torch.load(out / "pytorch_model.bin")
    assert set(got) == set(hf)
    for k in hf:
        torch.testing.assert_close(got[k], hf[k], msg=k)
    cfg = json.load(open(out / "config.json"))
    assert cfg["num_hidden_layers"] == layers and cfg["intermediate_size"] == ffn and cfg["vocab_size"] == vocab


def test_generate_petreloss_conf(tmp_path):
    tool = _tool("generate_petreloss_conf")
    out = tmp_path / "petreloss.conf"
    tool.main(["--access_key", "AK", "--secret_key", "SK", "--host_base", "http://ceph:80", "--cluster", "c1",
               "--out", str(out)])
    import configparser
    cp = configparser.ConfigParser()
    cp.read(out)
    assert cp["DEFAULT"]["default_cluster"] == "c1" and cp["c1"]["access_key"] == "AK" and cp["c1"]["host_base"].endswith(":80")


def test_build_index_mmap_from_config(tmp_path):
    """The offline cache builder reads the dataset block of a training YAML and leaves a reusable .bin/.idx cache."""
    tool = _tool("build_index_mmap")
    lines = [json.dumps({"text": "doc %d " % i + "w" * (5 + i % 7)}) for i in range(40)]
    jf = tmp_path / "d.jsonl"
    jf.write_text("\n".join(lines) + "\n")
    cfg = f"""
tokenizer:
  type: SimpleTokenizer
  kwargs: {{}}
data:
  train:
    dataset:
      type: mmap_index_json
      kwargs:
        data_root: {tmp_path}
        seed: 1
        total_samples: 20
        max_seq_length: 32
        json_file: {jf}
        cache_worker: 2
        transformer:
          - type: sense_tokenization
            kwargs: {{max_seq_length: 4096, parser_type: base}}
"""
    y = tmp_path / "cfg.yaml"
    y.write_text(cfg)
    tool.main(["--config", str(y)])
    cache = list((tmp_path / "train_data_cache").iterdir())
    assert any(p.name.endswith(".bin") for p in cache) and any(p.name.endswith(".idx") for p in cache)
    # a dataset built afterwards finds the cache (no rebuild: the .bin keeps its mtime)
    from easyllm_b200.config import load_yaml
    from easyllm_b200.data import build_dataset, build_tokenizer
    c = load_yaml(str(y))
    before = {p.name: p.stat().st_mtime_ns for p in cache}
    ds = build_dataset(c["data"]["train"]["dataset"], build_tokenizer(c["tokenizer"]))
    assert len(ds) >= 20 and ds[0]["input_ids"].shape[0] == 33
    after = {p.name: p.stat().st_mtime_ns for p in (tmp_path / "train_data_cache").iterdir()}
    assert all(after[k] == v for k, v in before.items() if k.endswith(".bin"))


def test_medusa_runner_trains_heads_only_and_answers_questions(tmp_path):
    """MedusaRunner end to end on CPU: only the extra heads train, the checkpoint is ``medusa_lm_head.pth``, and
    inference over a question file writes one result per question with acceptance statistics."""
    import copy
    import json
    import os
    from easyllm_b200.config import load_yaml, parse_args
    from easyllm_b200.runners.medusa_runner import MedusaRunner
    cfg_path = os.path.join(os.path.dirname(__file__), "..", "configs", "huggingface", "tiny_llama_cpu.yaml")
    cfg = load_yaml(cfg_path)
    with open(tmp_path / "d.jsonl", "w") as f:
        for i in range(32):
            f.write(json.dumps({"instruction": f"question number {i}", "input": "", "output": f"answer {i % 5}"}) + "\n")
    cfg["data"]["train"]["dataset"]["kwargs"]["json_file"] = str(tmp_path / "d.jsonl")
    cfg["saver"] = {"enabled": True, "save_path": str(tmp_path / "ck"), "save_interval": 3, "save_mode": "huggingface"}
    cfg["trainer"]["train_iters"] = 3
    cfg["hooks"] = [h for h in cfg.get("hooks", []) if h["type"] != "dynamic_checkpoint"]
    cfg["model"] = {"type": "medusa", "kwargs": {"base_model": copy.deepcopy(cfg["model"]), "medusa_num_heads": 2,
                                                  "medusa_num_layers": 1}}
    r = MedusaRunner(parse_args(["--config", cfg_path]), cfg, training=True)
    trainable = [n for n, p in r.model.named_parameters() if p.requires_grad]
    assert trainable and all(n.startswith("medusa_head") for n in trainable)
    base_before = {n: p.detach().clone() for n, p in r.model.base_model.named_parameters()}
    head_before = {n: p.detach().clone() for n, p in r.model.medusa_head.named_parameters()}
    r.train()
    assert all(torch.equal(p.detach().float(), base_before[n].float()) for n, p in r.model.base_model.named_parameters())
    assert any(not torch.equal(p.detach().float(), head_before[n].float()) for n, p in r.model.medusa_head.named_parameters())
    saved = tmp_path / "ck" / "checkpoint-3" / "medusa_lm_head.pth"
    assert saved.exists() and set(torch.load(saved)) == set(r.model.medusa_head.state_dict())

    with open(tmp_path / "q.jsonl", "w") as f:
        f.write(json.dumps({"instruction": "question number 1", "input": "", "output": "answer 1"}) + "\n")
        f.write(json.dumps({"instruction": "another", "input": " one", "output": "x"}) + "\n")
    cfg2 = copy.deepcopy(cfg)
    cfg2["infer_cfg"] = {"question_file": str(tmp_path / "q.jsonl"), "result_file": str(tmp_path / "res.jsonl")}
    cfg2["model"]["kwargs"]["medusa_head_name_or_path"] = str(saved)
    cfg2["infer_tokenization"] = {"type": "sense_tokenization", "kwargs": {
        "max_seq_length": 128, "parser_type": "simple_chat", "parser_kwargs": {"inference_mode": True}}}
    args = parse_args(["--config", cfg_path, "--inference", "--medusa-generate", "--medusa-max-steps", "4",
                       "--medusa-choices", "mc_sim_7b_3_head_top5"])
    r2 = MedusaRunner(args, cfg2, training=False)
    res = r2.infer()
    lines = [json.loads(l) for l in open(tmp_path / "res.jsonl")]
    assert len(res) == len(lines) == 2 and lines[1]["input"] == "another one" and lines[0]["answer"] == "answer 1"
    assert all(l["infos"]["count"] >= 1 and l["infos"]["accept_length"] >= l["infos"]["count"] for l in lines)
