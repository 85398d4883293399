"""Megatron runner on CPU through the task-specific data paths: SFT from json chat records, offline DPO pairs with
reference log-probabilities, mini-RLHF ranked answers (parser → collator → batch function → loss, from YAML)."""
import copy
import json
import os

from dist_utils import run_ranks

CFG = os.path.join(os.path.dirname(__file__), "..", "configs", "megatron", "tiny_llama_cpu.yaml")


def _run(rank, world, cfg, iters):
    from easyllm_b200.config import parse_args
    from easyllm_b200.runners.base_llm_runner import BaseRunner
    cfg = copy.deepcopy(cfg)
    cfg["trainer"]["train_iters"] = iters
    args = parse_args(["--config", CFG, "--launcher", "torch", "--distributed-backend", "gloo"])
    r = BaseRunner(args, cfg, training=True, base_type="train")
    seen = []
    orig = r.forward_step

    def rec(it):
        out = orig(it)
        seen.append({k: float(v) for k, v in out.items()})
        return out
    r.forward_step = rec
    r.train()
    return seen


def _base_cfg(tmp_path, parser_type, parser_kwargs=None):
    from easyllm_b200.config import load_yaml
    cfg = load_yaml(CFG)
    tok = {"type": "sense_tokenization", "kwargs": {"max_seq_length": 128, "parser_type": parser_type,
                                                    "parser_kwargs": parser_kwargs or {}}}
    cfg["data"]["train"]["dataset"] = {"type": "base_nlp_json", "kwargs": {
        "json_file": str(tmp_path / "d.jsonl"), "transformer": [tok], "json_type": "line"}}
    cfg["saver"]["save_path"] = str(tmp_path / "ck")
    cfg["saver"]["save_interval"] = 1000
    cfg["loader"]["load_path"] = None
    return cfg


def test_sft_from_chat_records(tmp_path):
    with open(tmp_path / "d.jsonl", "w") as f:
        for i in range(64):
            f.write(json.dumps({"messages": [{"role": "user", "content": f"say the number {i % 4}"},
                                             {"role": "assistant", "content": f"the number is {i % 4}"}]}) + "\n")
    cfg = _base_cfg(tmp_path, "simple_chat")
    cfg["data"]["train"]["batch_pipe"] = {"type": "json_batch_pipe", "kwargs": {}}
    seen = run_ranks(1, _run, cfg, 6)[0]
    assert len(seen) == 6 and all("lm_loss" in s for s in seen) and seen[-1]["lm_loss"] < seen[0]["lm_loss"]


def test_offline_dpo_pairs(tmp_path):
    good = [{"role": "user", "content": "pick a colour"}, {"role": "assistant", "content": "blue is calm"}]
    bad = [{"role": "user", "content": "pick a colour"}, {"role": "assistant", "content": "no"}]
    # per-token reference log-probabilities as `infer_logp` writes them: one value per token after the first
    from easyllm_b200.data import SimpleTokenizer, build_parser
    chat = build_parser("general_chat", dict(tokenizer=SimpleTokenizer(vocab_size=32000), max_seq_length=128))
    n_w, n_l = len(chat(good)["input_ids"]), len(chat(bad)["input_ids"])
    with open(tmp_path / "d.jsonl", "w") as f:
        for i in range(64):
            f.write(json.dumps({"yw": good, "yl": bad, "yw_logp": [-2.0] * (n_w - 1), "yl_logp": [-2.5] * (n_l - 1)}) + "\n")
    cfg = _base_cfg(tmp_path, "combine_dpo_general_chat")
    cfg["data"]["train"]["batch_pipe"] = {"type": "mini_rlhf_json_batch_pipe", "kwargs": {}}
    cfg["data"]["train"]["batch_collector"] = {"type": "mini_rlhf_batch", "kwargs": {"alignment": 4, "max_seq_length": 128}}
    cfg["data"]["train"]["micro_batch_size"] = 1
    cfg["data"]["train"]["batch_sampler"]["kwargs"]["micro_batch_size"] = 1
    cfg["data"]["train"]["batch_calculator"]["kwargs"].update(micro_batch_size=1, global_batch_size=2)
    cfg["data"]["train"]["global_batch_size"] = 2
    cfg["model"]["kwargs"]["loss_params"] = {"type": "dpo_loss", "kwargs": {"beta": 0.1}}
    seen = run_ranks(1, _run, cfg, 4)[0]
    assert len(seen) == 4
    keys = set(seen[0])
    assert any("loss" in k for k in keys), keys
    assert all(v == v for s in seen for v in s.values())                    # finite


def test_mini_rlhf_ranked_answers(tmp_path):
    with open(tmp_path / "d.jsonl", "w") as f:
        for i in range(64):
            f.write(json.dumps({"question": f"question {i % 3}? ", "answers": ["a good answer", "bad"],
                                "scores": [0.9, 0.1]}) + "\n")
    cfg = _base_cfg(tmp_path, "mini_rlhf")
    cfg["data"]["train"]["batch_pipe"] = {"type": "mini_rlhf_json_batch_pipe", "kwargs": {}}
    cfg["data"]["train"]["batch_collector"] = {"type": "mini_rlhf_batch", "kwargs": {"alignment": 8, "max_seq_length": 128}}
    cfg["data"]["train"]["micro_batch_size"] = 1
    cfg["data"]["train"]["batch_sampler"]["kwargs"]["micro_batch_size"] = 1
    cfg["data"]["train"]["batch_calculator"]["kwargs"].update(micro_batch_size=1, global_batch_size=2)
    cfg["data"]["train"]["global_batch_size"] = 2
    cfg["model"]["kwargs"]["loss_params"] = {"type": "mini_rlhf_entropy", "kwargs": {"sentense_pairs": 2}}
    seen = run_ranks(1, _run, cfg, 4)[0]
    assert len(seen) == 4 and all(v == v for s in seen for v in s.values())


def _interactive(rank, world, cfg):
    import builtins
    from easyllm_b200.config import parse_args
    from easyllm_b200.runners.base_llm_runner import BaseRunner
    from easyllm_b200.utils.log import default_logger
    cfg = copy.deepcopy(cfg)
    args = parse_args(["--config", CFG, "--launcher", "torch", "--distributed-backend", "gloo", "--inference",
                       "--generate-mode", "interactive", "--out-seq-length", "4", "--greedy"])
    r = BaseRunner(args, cfg, training=False, base_type="infer")
    script = iter(["hello there", "quit"])
    builtins.input = lambda *a: next(script)
    lines = []
    orig = default_logger.info
    default_logger.info = lambda m, *a, **k: (lines.append(str(m)), orig(m, *a, **k))
    try:
        r.generate()
    finally:
        default_logger.info = orig
    return r.config["data"]["data_types"], sorted(r.data_iterators), [l for l in lines if "EasyLLM:" in l]


def test_interactive_generation_from_a_training_config():
    """A config written for training (no ``data.infer`` block) still serves ``--inference``: the runner fills in the
    interactive defaults and does not build the training data."""
    from easyllm_b200.config import load_yaml
    cfg = load_yaml(CFG)
    cfg["loader"]["load_path"] = None
    cfg["infer_tokenization"] = {"type": "sense_tokenization", "kwargs": {
        "max_seq_length": 64, "parser_type": "simple_chat", "parser_kwargs": {"inference_mode": True}}}
    types, iters, replies = run_ranks(1, _interactive, cfg)[0]
    assert types == ["infer"] and iters == [] and len(replies) == 1


def _lora_train_and_logits(rank, world, save_dir):
    import torch
    from easyllm_b200.config import load_yaml, parse_args
    from easyllm_b200.runners.base_llm_runner import BaseRunner
    cfg = load_yaml(CFG)
    cfg["runtime"].update(tensor_model_parallel_size=2, pipeline_model_parallel_size=1, lora_mode=True)
    cfg["saver"]["save_path"] = save_dir
    cfg["trainer"]["train_iters"] = 3
    cfg["trainer"]["optimizer"]["kwargs"]["lr"] = 5.e-3          # large steps so the adapters clearly matter
    cfg["loader"]["load_path"] = None
    cfg["lora"] = {"lora_rank": 4, "lora_alpha": 8, "lora_dropout": 0.0,
                   "target_modules": ["q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj"],
                   # the full layer files are written too: they are the base model of this test
                   "saver": {"save_path": os.path.join(save_dir, "lora"), "only_save_trainable": False, "modules_to_save": []}}
    args = parse_args(["--config", CFG, "--launcher", "torch", "--distributed-backend", "gloo"])
    r = BaseRunner(args, cfg, training=True, base_type="train")
    r.train()
    r.model.eval()
    tok = (torch.arange(0, 40) * 13 % 32000).view(1, 40)
    with torch.no_grad():
        return r.model((tok, None, None), return_logits=True).detach()      # this rank's vocabulary shard


def _load_lora_tp1(rank, world, hf_base, mode, lora_path):
    import torch
    from easyllm_b200.ckpt.hf_import import load_llama_from_hf_format
    from easyllm_b200.config import load_yaml
    from easyllm_b200.models import build_model
    from easyllm_b200.models.lora import load_lora_ckpt_pretrained
    from easyllm_b200.data import build_tokenizer
    cfg = load_yaml(CFG)
    cfg_lora = {"lora_rank": 4, "lora_alpha": 8, "lora_dropout": 0.0,
                "target_modules": ["q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj"],
                "loader": {"load_path": lora_path, "load_mode": mode}}
    model = build_model(build_tokenizer(cfg["tokenizer"]), cfg, True, cfg_lora, base_type="train").eval()
    load_llama_from_hf_format(model, hf_base, "llama", worker=2)
    load_lora_ckpt_pretrained(cfg_lora, model)
    tok = (torch.arange(0, 40) * 13 % 32000).view(1, 40)
    with torch.no_grad():
        return model((tok, None, None), return_logits=True)


def _load_lora_tp1_modes(rank, world, hf_base, modes):
    return [_load_lora_tp1(rank, world, hf_base, mode, path) for mode, path in modes]


def test_lora_train_convert_merge_matches_the_trained_model(tmp_path):
    """The LoRA flow end to end at TP=2: train adapters with the Megatron runner, convert the base layer files and
    the adapter layer files to HF / peft format, merge them with the CLI tool, and get the trained model's logits back
    from a plain HuggingFace Llama."""
    import importlib.util
    import torch
    d = str(tmp_path / "ck")
    shards = run_ranks(2, _lora_train_and_logits, d)
    ours = torch.cat(shards, dim=-1)

    def tool(name):
        spec = importlib.util.spec_from_file_location(name, os.path.join(os.path.dirname(__file__), "..", "tools", name + ".py"))
        m = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(m)
        return m
    conv = tool("convert_ds_weight_to_hf_fast")
    geometry = ["--tp_size", "2", "--n_heads", "4", "--num_key_value_heads", "4", "--norm_eps", "1e-5"]
    conv.main(["--input_dir", os.path.join(d, "global_step3"), "--output_dir", str(tmp_path / "hf_base")] + geometry)
    conv.main(["--input_dir", os.path.join(d, "lora", "global_step3"), "--output_dir", str(tmp_path / "adapter"),
               "--lora_mode"] + geometry)
    assert os.path.exists(tmp_path / "adapter" / "adapter_model.bin")
    tool("merge_base_model_with_lora").main(["--base_model", str(tmp_path / "hf_base"), "--lora_model",
                                             str(tmp_path / "adapter"), "--output_dir", str(tmp_path / "merged")])
    from transformers import LlamaForCausalLM
    tok = (torch.arange(0, 40) * 13 % 32000).view(1, 40)
    merged = LlamaForCausalLM.from_pretrained(str(tmp_path / "merged"), torch_dtype=torch.float32,
                                              attn_implementation="eager")(input_ids=tok).logits
    base = LlamaForCausalLM.from_pretrained(str(tmp_path / "hf_base"), torch_dtype=torch.float32,
                                            attn_implementation="eager")(input_ids=tok).logits
    assert torch.allclose(ours, merged, atol=5e-4, rtol=1e-3), (ours - merged).abs().max()
    assert (ours - base).abs().max() > 10 * (ours - merged).abs().max()      # the adapters are what closes the gap
    # the adapters trained at TP 2 load into a TP 1 model, from the layer files (re-sharded) and from the peft folder
    modes = (("deepspeed", os.path.join(d, "lora", "global_step3")), ("huggingface", str(tmp_path / "adapter")))
    for (mode, _), again in zip(modes, run_ranks(1, _load_lora_tp1_modes, str(tmp_path / "hf_base"), modes)[0]):
        assert torch.allclose(again, ours, atol=5e-4, rtol=1e-3), (mode, (again - ours).abs().max())


def _pretrain_bin(rank, world, cfg, iters):
    from easyllm_b200.config import parse_args
    from easyllm_b200.runners.base_llm_runner import BaseRunner
    cfg = copy.deepcopy(cfg)
    cfg["runtime"].update(tensor_model_parallel_size=1, pipeline_model_parallel_size=world)
    cfg["trainer"]["train_iters"] = iters
    args = parse_args(["--config", CFG, "--launcher", "torch", "--distributed-backend", "gloo"])
    r = BaseRunner(args, cfg, training=True, base_type="train")
    seen, batches = [], []
    orig_fn = r.batch_pipe_func["train"]

    def spy(data):
        out = orig_fn(data)
        batches.append([tuple(t.shape) if hasattr(t, "shape") else None for t in out[0]])
        return out
    r.batch_pipe_func["train"] = spy
    r.engine.set_batch_fn(spy)
    orig = r.forward_step

    def rec(it):
        out = orig(it)
        seen.append(float(out["lm_loss"]))
        return out
    r.forward_step = rec
    r.train()
    return seen, batches


def test_packed_pretraining_from_token_bins_over_two_pipeline_stages(tmp_path):
    """jsonl → token bins (the offline tool) → pretrain_bin dataset → packed batches with per-document position
    ids and cu_seqlens → two pipeline stages; the loss is finite and falls on a repetitive corpus."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("bpb", os.path.join(os.path.dirname(__file__), "..", "tools",
                                                                      "build_pretrain_bin.py"))
    tool = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(tool)
    src = tmp_path / "docs.jsonl"
    src.write_text("\n".join(json.dumps({"content": "the quick brown fox jumps over the lazy dog. " * (1 + i % 3)})
                             for i in range(400)))
    tool.main(["--tokenizer_type", "SimpleTokenizer", "--jsonl", str(src), "--out_dir", str(tmp_path / "bins"),
               "--bin_size", "8192", "--workers", "1"])
    from easyllm_b200.config import load_yaml
    cfg = load_yaml(CFG)
    tok = {"type": "sense_tokenization", "kwargs": {"max_seq_length": 128, "parser_type": "pretrain_bin", "parser_kwargs": {}}}
    tr = cfg["data"]["train"]
    tr["dataset"] = {"type": "pretrain_bin", "kwargs": {"folders": str(tmp_path / "bins"), "seq_length": 128,
                                                         "bin_size": 8192, "transformer": [tok]}}
    tr["batch_collector"] = {"type": "batch_align", "kwargs": {"alignment": 8, "max_seq_length": 128, "pretrain": True,
                                                               "offset_label": True}}
    tr["batch_pipe"] = {"type": "flash_batch_pipe", "kwargs": {"eod_mask_loss": True, "pretrain": True}}
    cfg["saver"]["save_path"] = str(tmp_path / "ck")
    cfg["saver"]["save_interval"] = 1000
    cfg["loader"]["load_path"] = None
    cfg["trainer"]["optimizer"]["kwargs"]["lr"] = 2.e-3
    res = run_ranks(2, _pretrain_bin, cfg, 8)
    losses = res[1][0] or res[0][0]                     # the last stage records the loss
    assert len(losses) == 8 and all(l == l for l in losses) and losses[-1] < losses[0]
    first_stage_batches = res[0][1]
    # (tokens, position_ids, mask, cu_seqlens): documents are packed, so cu_seqlens has more than two entries
    assert first_stage_batches and len(first_stage_batches[0]) == 4 and first_stage_batches[0][3][0] > 2


def _infer_modes(rank, world, cfg, mode, extra):
    from easyllm_b200.config import parse_args
    from easyllm_b200.runners.base_llm_runner import BaseRunner
    cfg = copy.deepcopy(cfg)
    args = parse_args(["--config", CFG, "--launcher", "torch", "--distributed-backend", "gloo", "--inference",
                       "--generate-mode", mode, "--out-seq-length", "4", "--greedy"] + extra)
    r = BaseRunner(args, cfg, training=False, base_type="infer")
    r.generate()
    return True


def test_runner_eval_and_logp_modes_feed_offline_dpo(tmp_path):
    """``--generate-mode eval`` answers a question file; ``--generate-mode logp`` writes per-token label log-probs of a
    dataset, in the form the offline-DPO parser consumes as reference scores."""
    from easyllm_b200.config import load_yaml
    from easyllm_b200.data import SimpleTokenizer, build_parser
    cfg = load_yaml(CFG)
    cfg["loader"]["load_path"] = None
    cfg["infer_tokenization"] = {"type": "sense_tokenization", "kwargs": {
        "max_seq_length": 64, "parser_type": "simple_chat", "parser_kwargs": {"inference_mode": True}}}
    with open(tmp_path / "q.jsonl", "w") as f:
        f.write(json.dumps({"instruction": "name a colour", "input": "", "output": "blue"}) + "\n")
        f.write(json.dumps({"instruction": "name a", "input": " fruit", "output": "pear"}) + "\n")
    cfg["infer_cfg"] = {"eval_task": "base", "question_file": str(tmp_path / "q.jsonl"), "result_file": str(tmp_path / "r.jsonl")}
    assert run_ranks(1, _infer_modes, cfg, "eval", [])[0]
    rows = [json.loads(l) for l in open(tmp_path / "r.jsonl")]
    assert len(rows) == 2 and rows[1]["input"] == "name a fruit" and rows[0]["gold"] == "blue" and "raw_output" in rows[0]

    # logp over a chat dataset
    conv = [{"role": "user", "content": "pick a colour"}, {"role": "assistant", "content": "blue is calm"}]
    with open(tmp_path / "d.jsonl", "w") as f:
        for _ in range(4):
            f.write(json.dumps(conv) + "\n")
    tok = {"type": "sense_tokenization", "kwargs": {"max_seq_length": 128, "parser_type": "general_chat",
                                                    "parser_kwargs": {"only_last_answer": True}}}
    cfg2 = copy.deepcopy(cfg)
    train = cfg2["data"]["train"]
    cfg2["data"] = {"data_types": ["infer"], "infer": dict(
        train, infer_type="logp", micro_batch_size=1, global_batch_size=1,
        dataset={"type": "base_nlp_json", "kwargs": {"json_file": str(tmp_path / "d.jsonl"), "transformer": [tok],
                                                      "json_type": "line"}},
        batch_sampler={"type": "megatron_pretrain", "kwargs": {"micro_batch_size": 1, "drop_last": True}},
        batch_collector={"type": "batch_align", "kwargs": {"alignment": 1, "max_seq_length": 128}},
        batch_pipe={"type": "json_batch_pipe", "kwargs": {}},
        batch_calculator={"type": "constant_num", "kwargs": {"global_batch_size": 1, "micro_batch_size": 1}})}
    assert run_ranks(1, _infer_modes, cfg2, "logp", ["--logp-file", str(tmp_path / "logp.jsonl")])[0]
    lines = [json.loads(l) for l in open(tmp_path / "logp.jsonl")]
    chat = build_parser("general_chat", dict(tokenizer=SimpleTokenizer(vocab_size=32000), max_seq_length=128,
                                             only_last_answer=True))
    n = len(chat(conv)["input_ids"])
    assert len(lines) == 4 and all(len(l["logp"]) == n - 1 for l in lines)     # one value per token after the first
    assert all(v <= 0 for v in lines[0]["logp"]) and lines[0]["logp"] == lines[1]["logp"]
    # and those lists are exactly what the DPO parser takes as yw_logp / yl_logp
    dpo = build_parser("combine_dpo_general_chat", dict(tokenizer=SimpleTokenizer(vocab_size=32000), max_seq_length=128))
    pair = dpo({"yw": conv, "yl": conv, "yw_logp": lines[0]["logp"], "yl_logp": lines[1]["logp"]})
    assert pair["scores"][0] == pair["scores"][1] < 0


def test_sft_from_the_mmap_index_dataset(tmp_path):
    """The Megatron-style indexed dataset (tokenise once into .bin/.idx, sample fixed-length windows through the
    native location index) feeding the runner, as in the mmap SFT config."""
    with open(tmp_path / "d.jsonl", "w") as f:
        for i in range(200):
            f.write(json.dumps({"messages": [{"role": "user", "content": f"count to {i % 5}"},
                                             {"role": "assistant", "content": " ".join(str(k) for k in range(i % 5 + 1))}]}) + "\n")
    from easyllm_b200.config import load_yaml
    cfg = load_yaml(CFG)
    tok = {"type": "sense_tokenization", "kwargs": {"max_seq_length": 4096, "parser_type": "simple_chat",
                                                    "parser_kwargs": {"keep_all_keys": False}}}
    cfg["data"]["train"]["dataset"] = {"type": "mmap_index_json", "kwargs": {
        "data_root": str(tmp_path), "seed": 7, "total_samples": 64, "max_seq_length": 128,
        "json_file": str(tmp_path / "d.jsonl"), "transformer": [tok], "cache_location_builder": "cpp"}}
    cfg["saver"]["save_path"] = str(tmp_path / "ck")
    cfg["saver"]["save_interval"] = 1000
    cfg["loader"]["load_path"] = None
    cfg["trainer"]["optimizer"]["kwargs"]["lr"] = 2.e-3
    seen = run_ranks(1, _run, cfg, 6)[0]
    assert len(seen) == 6 and all(s["lm_loss"] == s["lm_loss"] for s in seen) and seen[-1]["lm_loss"] < seen[0]["lm_loss"]
    cache = os.listdir(tmp_path / "train_data_cache")
    assert any(n.endswith(".bin") for n in cache) and any(n.endswith(".idx") for n in cache)


def _other_optimizers(rank, world, kinds):
    """Both runners with optimizer types other than the native fused Adam, from their YAML."""
    import torch
    from easyllm_b200.config import load_yaml, parse_args
    from easyllm_b200.parallel.grid import initialize_model_parallel
    from easyllm_b200.runners.base_llm_runner import BaseRunner
    from easyllm_b200.runners.hf_runner import HFRunner
    hf_cfg_path = os.path.join(os.path.dirname(CFG), "..", "huggingface", "tiny_llama_cpu.yaml")
    out = {}
    for kind, kwargs in kinds:
        cfg = load_yaml(CFG)
        cfg["runtime"].update(tensor_model_parallel_size=1, pipeline_model_parallel_size=world)
        cfg["trainer"]["train_iters"] = 5
        cfg["trainer"]["optimizer"] = {"type": kind, "kwargs": dict(kwargs)}
        cfg["saver"]["save_path"] = None
        cfg["loader"]["load_path"] = None
        args = parse_args(["--config", CFG, "--launcher", "torch", "--distributed-backend", "gloo"])
        r = BaseRunner(args, cfg, training=True, base_type="train")
        before = [p.detach().clone() for p in r.model.parameters()]
        losses = []
        orig = r.forward_step

        def rec(it, _orig=orig, _l=losses):
            o = _orig(it)
            _l.append(float(o["lm_loss"]))
            return o
        r.forward_step = rec
        r.train()
        moved = max(float((p.detach() - b).abs().max()) for p, b in zip(r.model.parameters(), before))
        out[kind] = (type(r.optimizer).__name__, type(getattr(r.optimizer, "inner", None)).__name__, losses,
                     r.engine.get_global_grad_norm(), moved)
    return out


def test_runner_drives_non_native_optimizers_over_two_pipeline_stages():
    kinds = [("SophiaG", {"lr": 2e-4, "betas": [0.9, 0.99], "rho": 0.04, "weight_decay": 0.0}),
             ("Adam8bit", {"lr": 1e-3, "min_8bit_size": 1024, "block_size": 256}),
             ("SGD", {"lr": 0.05, "momentum": 0.9})]
    res = run_ranks(2, _other_optimizers, kinds)
    last = res[1]                                       # the last stage records the loss
    for kind, inner in (("SophiaG", "SophiaG"), ("Adam8bit", "Adam8bit"), ("SGD", "SGD")):
        wrapper, inner_name, losses, norm, moved = last[kind]
        assert wrapper == "TorchOptimizerAdapter" and inner_name == inner
        assert len(losses) == 5 and all(l == l and l < 12 for l in losses), (kind, losses)
        assert norm is not None and norm > 0 and moved > 0 and res[0][kind][4] > 0       # both stages were updated
