"""save (layer files, TP=2) → DS→HF converter → transformers.LlamaForCausalLM forward parity,
HF import back into a TP=1 model, and engine resume (bitwise continuation)."""
import os

import torch

from dist_utils import run_ranks

TINY = dict(num_layers=2, hidden_size=256, num_attention_heads=4, num_kv_attention_heads=2, intermediate_size=688,
            vocab_size=32000, layer_norm_params={"kwargs": {"eps": 1e-5}}, checkpoint_activations=False)


def _make_engine(tp=1, pp=1, stage=0, world=1, seed=0):
    from easyllm_b200.parallel.grid import initialize_model_parallel
    from easyllm_b200.parallel.rng import set_random_seed
    from easyllm_b200.models import llama_custom
    from easyllm_b200.optim import ZeroOptimizer, IterBaseAnnealingLR
    from easyllm_b200.engine import PipelineEngine
    if world > 1:
        initialize_model_parallel(tp, pp)
    set_random_seed(seed + 1)
    model = llama_custom(**TINY)
    opt = ZeroOptimizer(model.named_parameters(), lr=1e-3, adamw=False, stage=stage)
    sched = IterBaseAnnealingLR(opt, max_lr=1e-3, min_lr=1e-5, decay_style="cosine", lr_warmup_iters=1,
                                lr_decay_iters=10, global_batch_size=2)
    return PipelineEngine(model, opt, sched, {"train_micro_batch_size_per_gpu": 2, "gradient_accumulation_steps": 1})


def _save_tp2(rank, world, out_dir):
    from easyllm_b200.data.synthetic import synthetic_batches
    eng = _make_engine(tp=2, world=world)
    it = synthetic_batches(32000, 64, 2, seed=0)
    eng.train_batch(it)
    eng.save_checkpoint(out_dir, tag="global_step1", client_state={"iteration": 1, "samples": 2, "tokens": 128})
    tok = torch.arange(0, 48).remainder(32000).view(1, 48) * 7 % 32000
    logits = eng.module((tok, None, None), return_logits=True)    # vocab-parallel logits of this rank
    return logits.detach()


def test_tp2_checkpoint_converts_to_hf_and_back(tmp_path):
    out = str(tmp_path / "ds")
    shards = run_ranks(2, _save_tp2, out)
    ckpt = os.path.join(out, "global_step1")
    names = sorted(os.listdir(ckpt))
    assert "layer_01-model_00-model_states.pt" in names and "layer_07-model_01-model_states.pt" in names
    assert "mp_rank_00_model_states.pt" in names and open(os.path.join(out, "latest")).read() == "global_step1"
    assert any(n.startswith("zero_pp_rank_0_mp_rank_0") for n in names)
    # converter CLI (same flags as the reference tool)
    import importlib.util
    spec = importlib.util.spec_from_file_location("conv", os.path.join(os.path.dirname(__file__), "..", "tools",
                                                                       "convert_ds_weight_to_hf_fast.py"))
    conv = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(conv)
    hf_dir = str(tmp_path / "hf")
    conv.main(["--input_dir", ckpt, "--output_dir", hf_dir, "--tp_size", "2", "--n_heads", "4",
               "--num_key_value_heads", "2", "--norm_eps", "1e-5"])
    from transformers import LlamaForCausalLM
    hf = LlamaForCausalLM.from_pretrained(hf_dir, torch_dtype=torch.float32, attn_implementation="eager")
    tok = torch.arange(0, 48).remainder(32000).view(1, 48) * 7 % 32000
    ref = hf(input_ids=tok).logits
    ours = torch.cat(shards, dim=-1)
    assert torch.allclose(ours, ref, atol=2e-4, rtol=1e-4)
    # and back: HF → TP=1 model
    from easyllm_b200.models import llama_custom
    from easyllm_b200.ckpt.hf_import import load_llama_from_hf_format
    m = llama_custom(**TINY)
    load_llama_from_hf_format(m, hf_dir, "llama")
    assert torch.allclose(m((tok, None, None), return_logits=True), ref, atol=2e-4, rtol=1e-4)


def test_resume_continues_bitwise(tmp_path):
    from easyllm_b200.data.synthetic import synthetic_batches
    eng = _make_engine()
    it = synthetic_batches(32000, 64, 2, seed=3)
    l1 = [float(eng.train_batch(it)) for _ in range(2)]
    eng.save_checkpoint(str(tmp_path), client_state={"iteration": 2})
    l2 = [float(eng.train_batch(it)) for _ in range(2)]
    eng2 = _make_engine(seed=5)           # different init: everything must come from the files
    _, client = eng2.load_checkpoint(str(tmp_path))
    assert client["iteration"] == 2 and eng2.global_steps == 2
    it2 = synthetic_batches(32000, 64, 2, seed=3, start=2)
    l3 = [float(eng2.train_batch(it2)) for _ in range(2)]
    assert l3 == l2, (l2, l3)


def test_truncated_file_is_reported(tmp_path):
    eng = _make_engine()
    eng.save_checkpoint(str(tmp_path), tag="t")
    p = os.path.join(str(tmp_path), "t", "layer_03-model_00-model_states.pt")
    with open(p, "r+b") as f:
        f.truncate(100)
    try:
        eng.load_checkpoint(str(tmp_path))
    except RuntimeError as e:
        assert "unreadable" in str(e)
    else:
        raise AssertionError("truncated checkpoint was accepted")


def _save_pp2(rank, world, out_dir):
    from easyllm_b200.data.synthetic import synthetic_batches
    eng = _make_engine(pp=2, world=world)
    it = synthetic_batches(32000, 64, 2, seed=0)
    eng.train_batch(it)
    eng.save_checkpoint(out_dir, tag="global_step1", client_state={"iteration": 1})
    tok = torch.arange(0, 48).remainder(32000).view(1, 48) * 7 % 32000
    with torch.no_grad():
        out = eng.forward_tokens(tok, torch.arange(48).view(1, 48))      # logits on the last stage, None elsewhere
    return None if out is None else out.detach().float()


def test_checkpoint_written_with_pp2_loads_into_pp1(tmp_path):
    """Layer files are indexed by the position in the layer list, not by stage: a checkpoint saved by a 2-stage
    pipeline restores the weights of a single-process model (restart with another pipeline size)."""
    out = str(tmp_path / "ds")
    want = [r for r in run_ranks(2, _save_pp2, out) if r is not None][0]
    names = sorted(os.listdir(os.path.join(out, "global_step1")))
    assert {"layer_01-model_00-model_states.pt", "layer_03-model_00-model_states.pt", "layer_04-model_00-model_states.pt",
            "layer_06-model_00-model_states.pt", "layer_07-model_00-model_states.pt"} <= set(names)
    eng = _make_engine(seed=9)                       # different init: the weights must come from the files
    _, client = eng.load_checkpoint(out, load_module_only=True)
    assert client["iteration"] == 1
    tok = torch.arange(0, 48).remainder(32000).view(1, 48) * 7 % 32000
    with torch.no_grad():
        got = eng.module((tok, None, None), return_logits=True).float()
    assert torch.allclose(got.view(-1), want.view(-1), atol=1e-5), (got.view(-1) - want.view(-1)).abs().max()


def _engine_dp(world, grad_accum, seed=0):
    from easyllm_b200.parallel.grid import initialize_model_parallel
    from easyllm_b200.parallel.rng import set_random_seed
    from easyllm_b200.models import llama_custom
    from easyllm_b200.optim import ZeroOptimizer, IterBaseAnnealingLR
    from easyllm_b200.engine import PipelineEngine
    if world > 1:
        initialize_model_parallel(1, 1)
    set_random_seed(seed + 1)
    model = llama_custom(**TINY)
    opt = ZeroOptimizer(model.named_parameters(), lr=1e-3, stage=1, weight_decay=0.1, grad_clip=1.0)
    sched = IterBaseAnnealingLR(opt, max_lr=1e-3, min_lr=1e-5, decay_style="cosine", lr_warmup_iters=1,
                                lr_decay_iters=10, global_batch_size=4)
    return PipelineEngine(model, opt, sched, {"train_micro_batch_size_per_gpu": 2,
                                              "gradient_accumulation_steps": grad_accum})


def _train_dp2_save(rank, world, out_dir):
    from easyllm_b200.data.synthetic import synthetic_batches
    eng = _engine_dp(world, 1)
    it = synthetic_batches(32000, 64, 2, seed=7)
    for _ in range(2):
        eng.train_batch(it)
    eng.save_checkpoint(out_dir, client_state={"iteration": 2})
    return float(eng.train_batch(it))


def test_zero1_state_saved_with_dp2_resumes_on_one_rank(tmp_path):
    """The ZeRO-1 optimizer shards of a 2-rank run are re-assembled by parameter name when the data-parallel size
    changed: one rank with two accumulation steps continues with the same loss as the 2-rank run."""
    from easyllm_b200.data.synthetic import synthetic_batches
    out = str(tmp_path / "ds")
    third = run_ranks(2, _train_dp2_save, out)
    assert abs(third[0] - third[1]) < 1e-6
    eng = _engine_dp(1, 2, seed=11)                   # different init: weights and Adam state come from the files
    _, client = eng.load_checkpoint(out)
    assert client["iteration"] == 2 and eng.optimizer.step_count == 2
    it = synthetic_batches(32000, 64, 2, seed=7, start=4)      # 2 steps x 2 micro-batches of the global stream consumed
    loss = float(eng.train_batch(it))
    assert abs(loss - third[0]) < 2e-5, (loss, third)


def test_pipeline_module_names_used_by_checkpoint_helpers(tmp_path):
    """The DeepSpeed PipelineModule attribute names the reference's LoRA saver walks: the stage's layer list in
    order, the per-layer file path, the checkpoint engine; and the engine's ``_compute_loss`` switch."""
    from easyllm_b200.data.synthetic import synthetic_batches
    eng = _make_engine()
    m = eng.module
    funcs = m.forward_funcs
    assert len(funcs) == TINY["num_layers"] + 7 and funcs[0] == "to_float16" and funcs[2] == "transpose"
    assert funcs[1] is m.layers["1"] and funcs[3] is m.layers["3"] and funcs[-2] is m.layers[str(TINY["num_layers"] + 5)]
    assert m.checkpoint_parallel_write_pipeline is False
    path = m.ckpt_layer_path(str(tmp_path), 3)
    assert os.path.basename(path) == "layer_03-model_00-model_states.pt"
    m.checkpoint_engine.save({k: v.clone() for k, v in funcs[3].state_dict().items()}, path)
    eng.save_checkpoint(str(tmp_path / "full"), tag="t")
    ours = m.checkpoint_engine.load(path)
    full = torch.load(m.ckpt_layer_path(str(tmp_path / "full" / "t"), 3), weights_only=False)
    assert set(ours) == set(full) and all(torch.equal(ours[k], full[k]) for k in ours)
    # generation code of the reference flips _compute_loss and reads fwd_outputs
    eng._compute_loss = False
    out = eng.eval_batch(synthetic_batches(32000, 16, 2, seed=3))
    assert out.shape[:2] == (2, 16) and eng.fwd_outputs[0] is out
    eng._compute_loss = True
    assert eng.eval_batch(synthetic_batches(32000, 16, 2, seed=3)).dim() == 0


def _import_family(rank, world, path, pretrain_type, model_kw):
    from easyllm_b200.ckpt.hf_import import load_llama_from_hf_format
    from easyllm_b200.models import llama_custom
    from easyllm_b200.parallel.grid import initialize_model_parallel
    if world > 1:
        initialize_model_parallel(world, 1)
    m = llama_custom(**model_kw).eval()
    load_llama_from_hf_format(m, path, pretrain_type, worker=2)
    tok = (torch.arange(0, 24) * 5 % 300).view(1, 24)
    with torch.no_grad():
        return m((tok, None, None), return_logits=True)


def _import_families(rank, world, jobs):
    from easyllm_b200.parallel.grid import initialize_model_parallel
    if world > 1:
        initialize_model_parallel(world, 1)
    return [_import_family(rank, 1, *job) for job in jobs]      # the grid is set once for all of them


def test_family_checkpoints_import_into_the_megatron_model(tmp_path):
    """Qwen (fused c_attn with bias, w2 → gate, w1 → up), InternLM2 (GQA-interleaved wqkv, w1/w3/w2) and Baichuan
    (W_pack) checkpoints, written in each family's own key names, load into the 3D-parallel Llama model at TP 1 and
    TP 2 and reproduce the logits of the HF-style decoder they came from."""
    from easyllm_b200.models.hf_models import CausalLM, HFArch
    tok = (torch.arange(0, 24) * 5 % 300).view(1, 24)
    common = dict(vocab_size=304, hidden_size=64, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4)
    cases = [("qwen", "qwen", {"qkv_bias": True}, dict(transformer_layer_params={"attention_qkv_bias": True}), 4),
             ("internlm2", "internlm2", {"num_key_value_heads": 2}, {}, 2),
             ("baichuan", "baichuan", {}, {}, 4),
             ("llama", "llama", {"num_key_value_heads": 2}, {}, 2)]
    jobs = []
    for family, pretrain_type, arch_kw, model_extra, kv in cases:
        torch.manual_seed(1)
        src = CausalLM(HFArch(family=family, rms_norm_eps=1e-5, **common, **arch_kw)).eval()
        d = str(tmp_path / family)
        src.save_pretrained(d)
        with torch.no_grad():
            ref = src(tok)["logits"]
        model_kw = dict(num_layers=2, hidden_size=64, num_attention_heads=4, num_kv_attention_heads=kv,
                        intermediate_size=96, vocab_size=304, layer_norm_params={"kwargs": {"eps": 1e-5}},
                        checkpoint_activations=False, **model_extra)
        jobs.append((family, d, pretrain_type, model_kw, ref))
    ones = run_ranks(1, _import_families, [j[1:4] for j in jobs])[0]
    for (family, *_, ref), one in zip(jobs, ones):
        assert torch.allclose(one, ref, atol=2e-4, rtol=1e-4), (family, (one - ref).abs().max())
    sharded = [j for j in jobs if j[0] in ("qwen", "internlm2")]      # the fused / interleaved layouts, cut over TP
    twos = run_ranks(2, _import_families, [j[1:4] for j in sharded])
    for i, (family, *_, ref) in enumerate(sharded):
        two = torch.cat([twos[0][i], twos[1][i]], dim=-1)
        assert torch.allclose(two, ref, atol=2e-4, rtol=1e-4), (family, "tp2", (two - ref).abs().max())
