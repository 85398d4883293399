"""Megatron runner end to end on CPU/gloo from the YAML config: train, checkpoint, resume,
LoRA mode, and generation with the KV cache vs full recompute."""
import os

import torch

from dist_utils import run_ranks

CFG = os.path.join(os.path.dirname(__file__), "..", "configs", "megatron", "tiny_llama_cpu.yaml")


def _train(rank, world, save_dir, tp, pp, iters, resume, lora=False):
    from easyllm_b200.config import load_yaml, parse_args
    from easyllm_b200.runners.base_llm_runner import BaseRunner
    cfg = load_yaml(CFG)
    cfg["runtime"].update(tensor_model_parallel_size=tp, pipeline_model_parallel_size=pp)
    cfg["saver"]["save_path"] = save_dir
    cfg["trainer"]["train_iters"] = iters
    cfg["loader"]["load_path"] = save_dir if resume else None
    if lora:
        cfg["runtime"]["lora_mode"] = True
        cfg["lora"] = {"lora_rank": 4, "lora_alpha": 8, "lora_dropout": 0.0,
                       "target_modules": ["q_proj", "v_proj", "o_proj", "gate_proj", "down_proj"],
                       "saver": {"save_path": os.path.join(save_dir, "lora"), "only_save_trainable": True,
                                 "modules_to_save": []}}
    args = parse_args(["--config", CFG, "--launcher", "torch", "--distributed-backend", "gloo"])
    r = BaseRunner(args, cfg, training=True, base_type="train")
    losses = []
    orig = r.forward_step

    def rec(it):
        out = orig(it)
        losses.append(float(out["lm_loss"]))
        return out
    r.forward_step = rec
    r.train()
    n_train = sum(p.numel() for p in r.model.parameters() if p.requires_grad)
    return losses, r.start_iteration, r.consumed_train_samples, n_train


def test_train_save_resume_world2_pp2(tmp_path):
    d = str(tmp_path / "ck")
    full = run_ranks(2, _train, d, 1, 2, 4, False)[0]
    assert len(full[0]) == 4 and os.path.exists(os.path.join(d, "latest"))
    assert open(os.path.join(d, "latest")).read() == "global_step4"
    assert os.path.isdir(os.path.join(d, "global_step2"))
    # resume from iteration 4 and run 2 more: starts where the first run stopped
    res = run_ranks(2, _train, d, 1, 2, 6, True)[0]
    assert res[1] == 4 and len(res[0]) == 2 and res[2] == 6 * 4


def test_lora_mode_trains_only_adapters(tmp_path):
    d = str(tmp_path / "ck")
    losses, _, _, n_train = run_ranks(2, _train, d, 2, 1, 2, False, True)[0]
    assert len(losses) == 2 and 0 < n_train < 200_000
    files = os.listdir(os.path.join(d, "lora", "global_step2"))
    assert "adapter_config.json" in files and any(f.startswith("layer_03-model_01") for f in files)
    sd = torch.load(os.path.join(d, "lora", "global_step2", "layer_03-model_00-model_states.pt"))
    assert set(k.split(".")[-1] for k in sd) == {"lora_A_weight", "lora_B_weight"}
    assert "self_attn.q_proj.lora_A_weight" in sd and "mlp.down_proj.lora_B_weight" in sd


def _generate(rank, world, tp, pp):
    from easyllm_b200.parallel.grid import initialize_model_parallel
    from easyllm_b200.parallel.rng import set_random_seed
    from easyllm_b200.models import llama_custom
    from easyllm_b200.engine import PipelineEngine
    from easyllm_b200.data import SimpleTokenizer
    from easyllm_b200.infer.generation import Generator
    initialize_model_parallel(tp, pp)
    set_random_seed(5)
    torch.manual_seed(5)
    m = llama_custom(num_layers=2, hidden_size=128, num_attention_heads=4, num_kv_attention_heads=2,
                     intermediate_size=256, vocab_size=512, unpad_vocab_size=512, checkpoint_activations=False)
    eng = PipelineEngine(m, None, None, {})
    gen = Generator(eng, SimpleTokenizer(512))
    ctx = [[3, 17, 99, 250, 7], [9, 8, 7, 6, 5]]
    a = gen.generate_once(ctx, max_new_tokens=8, greedy=True, eos_id=-1)
    b = gen.generate_once(ctx, max_new_tokens=8, greedy=True, eos_id=-1, recompute=True)
    return a, b


def test_generation_kv_cache_equals_recompute_pp2():
    outs = run_ranks(2, _generate, 1, 2)
    for a, b in outs:
        assert a == b and len(a[0]) == 13
    assert outs[0][0] == outs[1][0]
