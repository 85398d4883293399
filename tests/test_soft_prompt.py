"""Prompt tuning and prefix tuning wrappers over the HF-style decoder (CPU)."""
import json

import torch


def _base(**kw):
    from easyllm_b200.models.hf_models import CausalLM, HFArch
    torch.manual_seed(0)
    a = HFArch(family="llama", vocab_size=97, hidden_size=64, intermediate_size=96, num_hidden_layers=2,
               num_attention_heads=4, num_key_value_heads=2, **kw)
    return CausalLM(a)


def test_prompt_tuning_matches_manual_embedding_concat_and_trains_only_the_prompt(tmp_path):
    from easyllm_b200.models.hf_models.soft_prompt import PromptTuning, load_adapter, save_adapter
    base = _base()
    m = PromptTuning(base, num_virtual_tokens=5, init_token_ids=[3, 4])
    emb = base.get_input_embeddings()
    assert torch.equal(m.prompt_embeddings.detach(), emb(torch.tensor([3, 4, 3, 4, 3])).detach())
    assert [n for n, p in m.named_parameters() if p.requires_grad] == ["prompt_embeddings"]
    ids = torch.randint(0, 97, (2, 9))
    logits = m(ids)["logits"]
    assert logits.shape == (2, 9, 97)
    x = torch.cat((m.prompt_embeddings.unsqueeze(0).expand(2, -1, -1), emb(ids)), 1)
    ref = base(torch.zeros(2, 14, dtype=torch.long), inputs_embeds=x)["logits"][:, 5:]
    assert torch.allclose(logits, ref, atol=1e-5)
    opt = torch.optim.Adam([m.prompt_embeddings], lr=0.05)
    losses = []
    for _ in range(8):
        loss = m(ids, labels=ids)["loss"]
        opt.zero_grad(); loss.backward(); opt.step()
        losses.append(float(loss.detach()))
    assert losses[-1] < losses[0] and all(p.grad is None for p in base.parameters())
    save_adapter(m, str(tmp_path))
    cfg = json.load(open(tmp_path / "adapter_config.json"))
    assert cfg["peft_type"] == "PROMPT_TUNING" and cfg["num_virtual_tokens"] == 5 and cfg["token_dim"] == 64
    again = load_adapter(base, str(tmp_path))
    assert torch.allclose(again(ids)["logits"], m(ids)["logits"], atol=1e-6)


def test_prefix_tuning_path_gradients_and_adapter_layout(tmp_path):
    from easyllm_b200.models.hf_models.soft_prompt import PrefixTuning, load_adapter, save_adapter
    base = _base()
    ids = torch.randint(0, 97, (2, 7))
    # an empty prefix is the base model: the pre-filled-cache path agrees with the packed training path
    empty = PrefixTuning(base, num_virtual_tokens=0)
    assert torch.allclose(empty(ids)["logits"], base(ids)["logits"], atol=1e-4)
    assert torch.allclose(empty(ids, labels=ids)["loss"], base(ids, labels=ids)["loss"], atol=1e-5)
    m = PrefixTuning(base, num_virtual_tokens=3)
    assert m.prefix.shape == (2, 2, 3, 2, 16)
    assert not torch.allclose(m(ids)["logits"], base(ids)["logits"], atol=1e-4)     # the prefix is attended to
    opt = torch.optim.Adam([m.prefix], lr=0.05)
    losses = []
    for _ in range(8):
        loss = m(ids, labels=ids)["loss"]
        opt.zero_grad(); loss.backward()
        assert m.prefix.grad.abs().sum() > 0
        opt.step()
        losses.append(float(loss.detach()))
    assert losses[-1] < losses[0] and all(p.grad is None for p in base.parameters())
    save_adapter(m, str(tmp_path))
    sd = torch.load(tmp_path / "adapter_model.bin")
    assert sd["prompt_embeddings"].shape == (3, 2 * 2 * 2 * 16)
    # peft's view of the tensor: [tokens, layers*2, heads, dim] with entry 2l the keys and 2l+1 the values of layer l
    view = sd["prompt_embeddings"].view(3, 4, 2, 16)
    assert torch.equal(view[:, 2], m.prefix.detach()[1, 0]) and torch.equal(view[:, 3], m.prefix.detach()[1, 1])
    again = load_adapter(base, str(tmp_path))
    assert torch.allclose(again(ids)["logits"], m(ids)["logits"], atol=1e-6)
    assert json.load(open(tmp_path / "adapter_config.json"))["peft_type"] == "PREFIX_TUNING"


def test_stand_alone_finetune_script_modes(tmp_path):
    """``open_hf_runner`` end to end on CPU: prompt tuning, prefix tuning and LoRA each train and write their
    adapter; full fine-tuning writes a loadable model."""
    import os
    from easyllm_b200.models.hf_models import CausalLM, HFArch
    from easyllm_b200.models.hf_models.soft_prompt import load_adapter
    from easyllm_b200.runners import open_hf_runner
    torch.manual_seed(0)
    a = HFArch(family="llama", vocab_size=32000, hidden_size=32, intermediate_size=64, num_hidden_layers=2,
               num_attention_heads=4)
    CausalLM(a).save_pretrained(str(tmp_path / "base"))
    with open(tmp_path / "d.jsonl", "w") as f:
        for i in range(16):
            f.write(json.dumps({"messages": [{"role": "user", "content": f"question {i}"},
                                             {"role": "assistant", "content": f"answer {i % 3}"}]}) + "\n")
    common = ["--model_name_or_path", str(tmp_path / "base"), "--family", "llama", "--tokenizer_type", "SimpleTokenizer",
              "--data_path", str(tmp_path / "d.jsonl"), "--model_max_length", "64", "--num_train_steps", "3",
              "--per_device_train_batch_size", "2", "--learning_rate", "1e-3", "--warmup_steps", "1"]
    open_hf_runner.main(common + ["--output_dir", str(tmp_path / "prompt"), "--tuning", "prompt", "--num_virtual_tokens", "4",
                                  "--prompt_init_text", "be brief"])
    open_hf_runner.main(common + ["--output_dir", str(tmp_path / "prefix"), "--tuning", "prefix", "--num_virtual_tokens", "3"])
    open_hf_runner.main(common + ["--output_dir", str(tmp_path / "lora"), "--use_lora"])
    open_hf_runner.main(common + ["--output_dir", str(tmp_path / "full")])
    base = CausalLM.from_pretrained(str(tmp_path / "base"), family="llama")
    ids = torch.randint(0, 255, (1, 6))
    for kind, n in (("prompt", 4), ("prefix", 3)):
        m = load_adapter(base, str(tmp_path / kind))
        assert m.n == n and m(ids)["logits"].shape == (1, 6, 32000)
    assert os.path.exists(tmp_path / "lora" / "adapter_model.bin") and os.path.exists(tmp_path / "lora" / "adapter_config.json")
    full = CausalLM.from_pretrained(str(tmp_path / "full"), family="llama")
    assert not torch.allclose(full(ids)["logits"], CausalLM.from_pretrained(str(tmp_path / "base"), family="llama")(ids)["logits"])


def test_soft_prompt_generation_agrees_with_full_recompute():
    """Decoding with the KV cache (virtual tokens in front) picks the same greedy tokens as re-running the whole
    wrapped model on the growing sequence."""
    from easyllm_b200.models.hf_models.soft_prompt import PrefixTuning, PromptTuning
    base = _base().eval()
    ids = torch.randint(0, 97, (2, 5))
    for m in (PromptTuning(base, 4), PrefixTuning(base, 3)):
        with torch.no_grad():
            (m.prompt_embeddings if hasattr(m, "prompt_embeddings") else m.prefix).mul_(20)   # make the prefix matter
        out = m.generate(ids, max_new_tokens=4, eos_token_id=None)
        assert out.shape == (2, 9) and torch.equal(out[:, :5], ids)
        cur = ids
        for t in range(4):
            nxt = m(cur)["logits"][:, -1].argmax(-1)
            assert torch.equal(nxt, out[:, 5 + t]), (type(m).__name__, t)
            cur = torch.cat((cur, nxt.unsqueeze(1)), 1)
        streamed = torch.stack(list(m.generate_stream(ids, max_new_tokens=4, eos_token_id=None)), 1)
        assert torch.equal(streamed, out[:, 5:])
