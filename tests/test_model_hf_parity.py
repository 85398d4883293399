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


def test_fp16_boundary_helpers():
    from easyllm_b200.models.fp16_module import Float16Module, float16_to_fp32, fp32_to_float16
    x = (torch.ones(2), [torch.ones(2, dtype=torch.int64), {"a": torch.ones(1)}], "s")
    y = fp32_to_float16(x)
    assert y[0].dtype == torch.bfloat16 and y[1][0].dtype == torch.int64 and y[1][1]["a"].dtype == torch.bfloat16 and y[2] == "s"
    z = float16_to_fp32(y)
    assert z[0].dtype == torch.float32 and z[1][0].dtype == torch.int64
    m = Float16Module(torch.nn.Linear(4, 3), bf16=True)
    out = m(torch.randn(5, 4))
    assert out.dtype == torch.float32 and m.module.weight.dtype == torch.bfloat16
    assert set(m.state_dict()) == {"weight", "bias"}


def test_scale_mask_softmax_wrapper():
    from easyllm_b200.models.fused_softmax import FusedScaleMaskSoftmax
    torch.manual_seed(0)
    s = torch.randn(2, 3, 5, 5)
    sm = FusedScaleMaskSoftmax(attn_mask_type="causal", scale=0.5)
    p = sm(s)
    assert torch.allclose(p.sum(-1), torch.ones(2, 3, 5), atol=1e-6)
    assert float(p[0, 0, 1, 2:].abs().max()) == 0.0                      # future positions carry no weight
    ref = torch.softmax((s * 0.5).masked_fill(torch.ones(5, 5, dtype=torch.bool).triu(1), float("-inf")), -1)
    assert torch.allclose(p, ref, atol=1e-6)
    pad = torch.zeros(2, 1, 1, 5, dtype=torch.bool); pad[:, :, :, -1] = True
    q = FusedScaleMaskSoftmax(attn_mask_type="padding", input_in_bf16=True)(s.bfloat16(), pad)
    assert q.dtype == torch.bfloat16 and float(q[..., -1].float().max()) < 1e-3
    # decoding step: one query row against a longer key axis sees every key
    one = FusedScaleMaskSoftmax(attn_mask_type="causal")(torch.randn(1, 1, 1, 7))
    assert float(one.min()) > 0
