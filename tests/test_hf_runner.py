"""HF-style runner on CPU/gloo: ZeRO-2 DP training from YAML, resume, family checkpoint IO,
LoRA merge, Dynamic Checkpoint selection."""
import json
import os

import torch

from dist_utils import run_ranks

CFG = os.path.join(os.path.dirname(__file__), "..", "configs", "huggingface", "tiny_llama_cpu.yaml")


def _write_data(path):
    with open(path, "w") as f:
        for i in range(64):
            f.write(json.dumps({"instruction": f"question number {i} about things", "input": "", "output": f"answer {i % 7}"}) + "\n")


def _train(rank, world, workdir, iters, resume):
    from easyllm_b200.config import load_yaml, parse_args
    from easyllm_b200.runners.hf_runner import HFRunner
    from easyllm_b200.parallel.grid import initialize_model_parallel
    initialize_model_parallel(1, 1)
    cfg = load_yaml(CFG)
    cfg["data"]["train"]["dataset"]["kwargs"]["json_file"] = os.path.join(workdir, "d.jsonl")
    cfg["saver"]["save_path"] = os.path.join(workdir, "ck")
    cfg["trainer"]["train_iters"] = iters
    if resume:
        cfg["loader"] = {"enabled": True, "load_path": os.path.join(workdir, "ck"), "load_mode": "deepspeed"}
    r = HFRunner(parse_args(["--config", CFG]), cfg, training=True)
    losses = []
    orig = r.engine.backward

    def rec(loss):
        losses.append(float(loss))
        return orig(loss)
    r.engine.backward = rec
    r.train()
    dc = [h for h in r._hooks if type(h).__name__ == "DynamicCheckpointHook"][0]
    return losses, r.start_iter, len(dc.mgr.cur_checkpoint_modules), len(dc.mgr.candidates)


def test_hf_runner_zero2_dp2_and_resume(tmp_path):
    _write_data(str(tmp_path / "d.jsonl"))
    outs = run_ranks(2, _train, str(tmp_path), 4, False)
    losses, start, n_ckpt, n_cand = outs[0]
    assert len(losses) == 8 and start == 0 and n_cand == 2 and n_ckpt in (0, 1, 2)
    assert losses[-1] < losses[0]
    assert os.path.exists(tmp_path / "ck" / "global_step4" / "mp_rank_00_model_states.pt")
    assert os.path.exists(tmp_path / "ck" / "checkpoint-4" / "pytorch_model.bin")
    res = run_ranks(2, _train, str(tmp_path), 6, True)[0]
    assert res[1] == 4 and len(res[0]) == 4


def test_family_checkpoint_roundtrip(tmp_path):
    from easyllm_b200.models.hf_models import CausalLM, HFArch
    ids = torch.randint(0, 300, (2, 10))
    for fam, extra in (("qwen", {}), ("internlm2", {"num_key_value_heads": 2}), ("baichuan2", {}),
                       ("baichuan2-13b", {"position": "alibi"}), ("internlm", {"qkv_bias": True, "o_bias": True})):
        torch.manual_seed(0)
        a = HFArch(family=fam, vocab_size=300, hidden_size=64, intermediate_size=96, num_hidden_layers=2,
                   num_attention_heads=4, qkv_bias=extra.pop("qkv_bias", fam == "qwen"), **extra)
        if fam.startswith("baichuan2"):
            a.norm_head = True
        m = CausalLM(a).eval()
        d = str(tmp_path / fam)
        m.save_pretrained(d)
        keys = torch.load(os.path.join(d, "pytorch_model.bin")).keys()
        probe = {"qwen": "transformer.h.0.attn.c_attn.weight", "internlm2": "model.layers.0.attention.wqkv.weight",
                 "baichuan2": "model.layers.0.self_attn.W_pack.weight", "baichuan2-13b": "model.layers.0.self_attn.W_pack.weight",
                 "internlm": "model.layers.0.self_attn.q_proj.bias"}[fam]
        assert probe in keys, (fam, list(keys)[:6])
        m2 = CausalLM.from_pretrained(d, family=fam).eval()
        with torch.no_grad():
            assert torch.allclose(m(ids)["logits"], m2(ids)["logits"], atol=1e-5), fam


def test_alibi_matches_cached_decode_and_lora_merge():
    from easyllm_b200.models.hf_models import CausalLM, HFArch
    from easyllm_b200.models.hf_models.lora import add_lora, merge_and_unload
    torch.manual_seed(1)
    a = HFArch(family="baichuan2-13b", position="alibi", vocab_size=200, hidden_size=64, intermediate_size=96,
               num_hidden_layers=2, num_attention_heads=4, eos_token_id=None)
    m = CausalLM(a).eval()
    ids = torch.randint(0, 200, (1, 9))
    out = m.generate(ids, max_new_tokens=5)
    with torch.no_grad():      # greedy decode with the cache must equal recomputing the full prefix
        for t in range(5):
            full = m(out[:, :9 + t])["logits"][:, -1].argmax(-1)
            assert int(full) == int(out[0, 9 + t])
    add_lora(m, {"r": 4, "lora_alpha": 8, "target_modules": ["q_proj", "down_proj"]})
    for mod in m.modules():
        if hasattr(mod, "lora_B"):
            torch.nn.init.normal_(mod.lora_B, std=0.05)
    assert sum(p.requires_grad for p in m.parameters()) == 2 * 2 * 2
    with torch.no_grad():
        before = m(ids)["logits"]
        after = merge_and_unload(m)(ids)["logits"]
    assert torch.allclose(before, after, atol=1e-4)


def test_fused_projection_aliases_adjacent_parameters():
    """q/k/v stored as separate (HF-named) parameters: once the optimizer has packed them into its flat buffer the
    fused projection aliases them instead of concatenating, and wgrad lands in the adjacent fp32 main_grad views."""
    from easyllm_b200 import ops
    from easyllm_b200.models.hf_models import CausalLM, HFArch
    from easyllm_b200.optim import ZeroOptimizer
    torch.manual_seed(0)
    a = HFArch(family="qwen", vocab_size=200, hidden_size=64, intermediate_size=96, num_hidden_layers=2,
               num_attention_heads=4, qkv_bias=True)
    m = CausalLM(a).train()
    att = m.model.layers[0].self_attn
    ws = (att.q_proj.weight, att.k_proj.weight, att.v_proj.weight)
    assert ops._adjacent_alias([w.detach() for w in ws]) is None          # separately allocated
    x = torch.randn(8, 64, requires_grad=True)
    y0 = ops._LinearParts.apply(x, None, *ws)
    y0.sum().backward()
    g0 = [w.grad.clone() for w in ws]
    dx0 = x.grad.clone()
    opt = ZeroOptimizer(m.named_parameters(), lr=1e-4, stage=0)
    assert ops._adjacent_alias([w.detach() for w in ws]) is not None
    assert ops._adjacent_alias([w.main_grad for w in ws]) is not None
    opt.zero_grad()
    x.grad = None
    y1 = ops._LinearParts.apply(x, None, *ws)
    y1.sum().backward()
    assert torch.allclose(y0, y1, atol=1e-6) and torch.allclose(dx0, x.grad, atol=1e-6)
    for w, g in zip(ws, g0):
        assert w.grad is None and torch.allclose(w.main_grad, g, atol=1e-5)


def _train_lora(rank, world, workdir):
    from easyllm_b200.config import load_yaml, parse_args
    from easyllm_b200.parallel.grid import initialize_model_parallel
    from easyllm_b200.runners.hf_runner import HFRunner
    initialize_model_parallel(1, 1)
    cfg = load_yaml(CFG)
    cfg["data"]["train"]["dataset"]["kwargs"]["json_file"] = os.path.join(workdir, "d.jsonl")
    cfg["saver"] = {"enabled": True, "save_path": os.path.join(workdir, "ck"), "save_mode": "huggingface", "save_interval": 3}
    cfg["trainer"]["train_iters"] = 3
    cfg["trainer"]["optimizer"]["kwargs"]["lr"] = 1.e-2
    cfg["hooks"] = [h for h in cfg.get("hooks", []) if h["type"] != "dynamic_checkpoint"]
    cfg["model"]["peft_model_cfg"] = {"r": 4, "lora_alpha": 8, "lora_dropout": 0.0, "target_modules": ["q_proj", "v_proj", "down_proj"]}
    r = HFRunner(parse_args(["--config", CFG]), cfg, training=True)
    base = {n: p.detach().clone() for n, p in r.model.named_parameters() if "lora_" not in n}
    trainable = [n for n, p in r.model.named_parameters() if p.requires_grad]
    r.train()
    frozen_ok = all(torch.equal(p.detach(), base[n]) for n, p in r.model.named_parameters() if "lora_" not in n)
    r.model.eval()
    ids = torch.arange(3, 19).view(1, 16)
    with torch.no_grad():
        logits = r.model(ids)["logits"].float()
    return trainable, frozen_ok, logits, {n.replace(".base.", "."): v for n, v in base.items()}


def test_hf_runner_lora_saves_an_adapter_that_merges_back(tmp_path):
    """LoRA through the HF runner's YAML (``model.peft_model_cfg``): only adapters train, the checkpoint is a peft
    adapter folder, and merging it into the untouched base weights reproduces the trained model."""
    from easyllm_b200.models.lora import merge_lora_into_hf_state
    _write_data(str(tmp_path / "d.jsonl"))
    trainable, frozen_ok, logits, base = run_ranks(1, _train_lora, str(tmp_path))[0]
    assert trainable and all("lora_" in n for n in trainable) and frozen_ok
    out = tmp_path / "ck" / "checkpoint-3"
    assert (out / "adapter_model.bin").exists() and (out / "adapter_config.json").exists()
    cfg = json.load(open(out / "adapter_config.json"))
    assert cfg["r"] == 4 and cfg["lora_alpha"] == 8 and sorted(cfg["target_modules"]) == ["down_proj", "q_proj", "v_proj"]
    adapter = torch.load(out / "adapter_model.bin")
    assert len(adapter) == 2 * 3 * 2                     # A and B for three projections in two layers
    merged = merge_lora_into_hf_state(base, adapter, cfg["lora_alpha"] / cfg["r"])
    from easyllm_b200.config import load_yaml
    from easyllm_b200.runners.hf_runner import build_hf_model
    model_cfg = load_yaml(CFG)["model"]
    plain = build_hf_model(model_cfg).float().eval()
    plain.load_state_dict({k: v.float() for k, v in merged.items()})
    with torch.no_grad():
        again = plain(torch.arange(3, 19).view(1, 16))["logits"]
    assert torch.allclose(again, logits, atol=1e-4, rtol=1e-4), (again - logits).abs().max()
    # `peft_model_cfg.peft_path` rebuilds the adapted model from the saved folder (for resuming or serving)
    served_cfg = dict(model_cfg, peft_model_cfg={"peft_path": str(out)})
    served = build_hf_model(served_cfg).float().eval()
    served.load_state_dict({(k if k in dict(served.named_parameters()) else k.replace(".weight", ".base.weight")): v.float()
                            for k, v in base.items()}, strict=False)
    with torch.no_grad():
        assert torch.allclose(served(torch.arange(3, 19).view(1, 16))["logits"], logits, atol=1e-4, rtol=1e-4)


def _hf_mode_roundtrip(rank, world, workdir, phase):
    from easyllm_b200.config import load_yaml, parse_args
    from easyllm_b200.parallel.grid import initialize_model_parallel
    from easyllm_b200.runners.hf_runner import HFRunner
    initialize_model_parallel(1, 1)
    cfg = load_yaml(CFG)
    cfg["data"]["train"]["dataset"]["kwargs"]["json_file"] = os.path.join(workdir, "d.jsonl")
    cfg["saver"] = {"enabled": True, "save_path": os.path.join(workdir, "ck"), "save_mode": "huggingface", "save_interval": 2}
    cfg["trainer"]["train_iters"] = 2
    cfg["hooks"] = [h for h in cfg.get("hooks", []) if h["type"] != "dynamic_checkpoint"]
    if phase != "train":
        cfg["loader"] = {"enabled": True, "load_path": os.path.join(workdir, "ck", "checkpoint-2"), "load_mode": "huggingface"}
    if phase == "lora":
        cfg["model"]["peft_model_cfg"] = {"r": 2, "lora_alpha": 4, "target_modules": ["q_proj", "o_proj"]}
    r = HFRunner(parse_args(["--config", CFG]), cfg, training=True)
    if phase == "train":
        r.train()
    r.model.eval()
    with torch.no_grad():
        return r.model(torch.arange(5, 21).view(1, 16))["logits"].float()


def _hf_mode_all_phases(rank, world, workdir):
    return tuple(_hf_mode_roundtrip(rank, world, workdir, phase) for phase in ("train", "load", "lora"))


def test_hf_mode_checkpoint_loads_back_also_under_lora_wrappers(tmp_path):
    """``save_mode: huggingface`` → ``loader.load_mode: huggingface``: the weights come back exactly, and they also
    reach the frozen projections of a model that has been wrapped for LoRA (fresh adapters start as a no-op)."""
    _write_data(str(tmp_path / "d.jsonl"))
    trained, loaded, wrapped = run_ranks(1, _hf_mode_all_phases, str(tmp_path))[0]
    assert torch.allclose(trained, loaded, atol=1e-5)
    assert torch.allclose(trained, wrapped, atol=1e-5)


def _hf_pretrain_bin(rank, world, workdir):
    from easyllm_b200.config import load_yaml, parse_args
    from easyllm_b200.parallel.grid import initialize_model_parallel
    from easyllm_b200.runners.hf_runner import HFRunner
    initialize_model_parallel(1, 1)
    cfg = load_yaml(CFG)
    tok = {"type": "sense_tokenization", "kwargs": {"max_seq_length": 128, "parser_type": "pretrain_bin"}}
    tr = cfg["data"]["train"]
    tr["dataset"] = {"type": "pretrain_bin", "kwargs": {"folders": os.path.join(workdir, "bins"), "seq_length": 128,
                                                         "bin_size": 4096, "transformer": [tok]}}
    tr["batch_collector"] = {"type": "batch_align", "kwargs": {"alignment": 8, "max_seq_length": 128, "pretrain": True}}
    cfg["saver"] = {"enabled": False}
    cfg["trainer"]["train_iters"] = 6
    cfg["trainer"]["optimizer"]["kwargs"]["lr"] = 3.e-3
    cfg["hooks"] = [h for h in cfg.get("hooks", []) if h["type"] != "dynamic_checkpoint"]
    r = HFRunner(parse_args(["--config", CFG]), cfg, training=True)
    losses, shapes = [], []
    orig_fwd = r.model.forward

    def fwd(*a, **k):
        shapes.append(None if k.get("cu_seqlens") is None else int(k["cu_seqlens"].numel()))
        return orig_fwd(*a, **k)
    r.model.forward = fwd
    orig = r.engine.backward

    def rec(loss):
        losses.append(float(loss))
        return orig(loss)
    r.engine.backward = rec
    r.train()
    return losses, shapes


def test_hf_runner_packed_pretraining_from_token_bins(tmp_path):
    """The HF runner on pre-tokenised bins: batches carry cu_seqlens / position ids of the packed documents down to
    the model's attention, and the loss falls."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("bpb", os.path.join(os.path.dirname(__file__), "..", "tools",
                                                                      "build_pretrain_bin.py"))
    tool = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(tool)
    (tmp_path / "docs.jsonl").write_text("\n".join(json.dumps({"content": "abc abc abc abc. " * (1 + i % 4)}) for i in range(300)))
    # the tiny config's vocabulary is 512: byte-level ids and the specials (256..258) fit
    tool.main(["--tokenizer_type", "SimpleTokenizer", "--jsonl", str(tmp_path / "docs.jsonl"), "--out_dir",
               str(tmp_path / "bins"), "--bin_size", "4096", "--workers", "1"])
    losses, shapes = run_ranks(1, _hf_pretrain_bin, str(tmp_path))[0]
    assert len(losses) >= 6 and losses[-1] < losses[0]
    assert shapes and all(s is not None and s > 2 for s in shapes)


def _hf_other_optimizer(rank, world, workdir):
    from easyllm_b200.config import load_yaml, parse_args
    from easyllm_b200.parallel.grid import initialize_model_parallel
    from easyllm_b200.runners.hf_runner import HFRunner
    initialize_model_parallel(1, 1)
    cfg = load_yaml(CFG)
    cfg["data"]["train"]["dataset"]["kwargs"]["json_file"] = os.path.join(workdir, "d.jsonl")
    cfg["saver"] = {"enabled": False}
    cfg["trainer"]["train_iters"] = 6
    cfg["trainer"]["optimizer"] = {"type": "Adam8bit", "kwargs": {"lr": 3e-3, "min_8bit_size": 1024, "block_size": 256}}
    cfg["hooks"] = [h for h in cfg.get("hooks", []) if h["type"] != "dynamic_checkpoint"]
    r = HFRunner(parse_args(["--config", CFG]), cfg, training=True)
    losses = []
    orig = r.engine.backward

    def rec(loss):
        losses.append(float(loss))
        return orig(loss)
    r.engine.backward = rec
    r.train()
    return type(r.optimizer.inner).__name__, losses


def test_hf_runner_uses_the_optimizer_type_of_its_yaml(tmp_path):
    """Two data-parallel ranks with ``trainer.optimizer.type: Adam8bit``: the wrapped optimizer is driven through
    the engine (gradient averaging over DP included) and the chat data is learnt."""
    _write_data(str(tmp_path / "d.jsonl"))
    res = run_ranks(2, _hf_other_optimizer, str(tmp_path))
    assert all(name == "Adam8bit" for name, _ in res)
    losses = res[0][1]
    assert len(losses) >= 6 and losses[-1] < losses[0]
