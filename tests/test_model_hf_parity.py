"""Tiny Llama (2 layers, hidden 256, 4 heads, FFN 688, eps 1e-5, vocab 32000) in fp32 on CPU:
loss and gradients must match transformers' LlamaForCausalLM carrying the same weights."""
import torch

from easyllm_b200.models import llama_custom

TINY = dict(num_layers=2, hidden_size=256, num_attention_heads=4, intermediate_size=688, vocab_size=32000,
            layer_norm_params={"kwargs": {"eps": 1e-5}}, checkpoint_activations=False)


def hf_twin(model, n_kv=4):
    from transformers import LlamaConfig, LlamaForCausalLM
    a = model.args
    cfg = LlamaConfig(vocab_size=a.vocab_size, hidden_size=a.hidden_size, intermediate_size=a.intermediate_size,
                      num_hidden_layers=a.num_layers, num_attention_heads=a.num_attention_heads,
                      num_key_value_heads=n_kv, rms_norm_eps=a.norm_eps, rope_theta=a.rope_base,
                      max_position_embeddings=4096, tie_word_embeddings=False, attention_bias=False)
    cfg._attn_implementation = "eager"
    hf = LlamaForCausalLM(cfg).float()
    sd = model.state_dict()
    L = a.num_layers
    new = {"model.embed_tokens.weight": sd["layers.1.word_embeddings.weight"],
           "model.norm.weight": sd[f"layers.{L + 4}.weight"],
           "lm_head.weight": sd[f"layers.{L + 5}.word_embeddings.weight"]}
    for i in range(L):
        for k, v in sd.items():
            pre = f"layers.{i + 3}."
            if k.startswith(pre):
                new[f"model.layers.{i}." + k[len(pre):]] = v
    missing, unexpected = hf.load_state_dict(new, strict=False)
    assert not unexpected, unexpected
    assert all("rotary" in m for m in missing), missing
    return hf


def test_loss_and_grads_match_hf():
    torch.manual_seed(0)
    m = llama_custom(**TINY)
    hf = hf_twin(m)
    g = torch.Generator().manual_seed(0)
    tok = torch.randint(0, 32000, (2, 128), generator=g)
    labels = torch.roll(tok, -1, 1)
    mask = torch.ones_like(labels)
    mask[:, -1] = 0
    loss = m((tok, None, None), (labels, mask))
    loss.backward()
    out = hf(input_ids=tok)
    ref = torch.nn.functional.cross_entropy(out.logits[:, :-1].reshape(-1, 32000), tok[:, 1:].reshape(-1))
    ref.backward()
    assert abs(loss.item() - ref.item()) < 1e-5
    ga = m.layers["3"].mlp.down_proj.weight.grad
    gb = hf.model.layers[0].mlp.down_proj.weight.grad
    assert torch.allclose(ga, gb, atol=1e-6, rtol=1e-4)
    gq = m.layers["4"].self_attn.qkv.weight.grad[:256]
    assert torch.allclose(gq, hf.model.layers[1].self_attn.q_proj.weight.grad, atol=1e-6, rtol=1e-4)


def test_gqa_and_packed_documents():
    torch.manual_seed(1)
    cfg = dict(TINY, num_kv_attention_heads=2)
    m = llama_custom(**cfg)
    hf = hf_twin(m, n_kv=2)
    tok = torch.randint(0, 32000, (1, 96))
    # two packed documents of 40 and 56 tokens: positions restart, attention does not cross
    pos = torch.cat((torch.arange(40), torch.arange(56))).unsqueeze(0)
    cu = torch.tensor([0, 40, 96], dtype=torch.int32)
    logits = m((tok, pos, None, cu), return_logits=True)
    a = hf(input_ids=tok[:, :40]).logits
    b = hf(input_ids=tok[:, 40:]).logits
    ref = torch.cat((a, b), dim=1)
    assert torch.allclose(logits, ref, atol=2e-4, rtol=1e-4)
