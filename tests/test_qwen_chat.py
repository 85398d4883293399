"""Qwen chat front end (ChatML context, stop words, chat / chat_stream) and the 8-bit decode KV cache."""
import base64

import pytest
import torch


def _tokenizer(tmp_path):
    pytest.importorskip("regex")
    from easyllm_b200.data.tokenizers_hf import QWenTokenizer
    toks = [bytes([i]) for i in range(256)] + [b"he", b"ll", b"hell", b"hello", b" w", b"or", b" wor"]
    with open(tmp_path / "qwen.tiktoken", "wb") as f:
        for r, t in enumerate(toks):
            f.write(base64.b64encode(t) + b" " + str(r).encode() + b"\n")
    return QWenTokenizer.from_pretrained(str(tmp_path))


def _model(vocab, **kw):
    from easyllm_b200.models.hf_models import CausalLM, HFArch
    torch.manual_seed(0)
    a = HFArch(family="qwen", vocab_size=vocab, hidden_size=64, intermediate_size=96, num_hidden_layers=2,
               num_attention_heads=4, qkv_bias=True, **kw)
    return CausalLM(a).eval()


def test_chatml_context_layout_and_history_window(tmp_path):
    from easyllm_b200.infer.qwen_chat import get_stop_words_ids, make_context
    tk = _tokenizer(tmp_path)
    text, ids = make_context(tk, "hello", history=[("q1", "a1"), ("q2", "a2")], system="sys")
    want = ("<|im_start|>system\nsys<|im_end|>\n<|im_start|>user\nq1<|im_end|>\n<|im_start|>assistant\na1<|im_end|>"
            "\n<|im_start|>user\nq2<|im_end|>\n<|im_start|>assistant\na2<|im_end|>"
            "\n<|im_start|>user\nhello<|im_end|>\n<|im_start|>assistant\n")
    assert text == want
    assert tk.decode(ids, skip_special_tokens=False) == want              # ids and text describe the same context
    assert ids.count(tk.im_start_id) == 7 and ids.count(tk.im_end_id) == 6
    # a window that only fits the newest turn drops the older one; a window below the system block drops both
    base = len(make_context(tk, "hello", system="sys")[1])
    one_turn = len(make_context(tk, "hello", history=[("q2", "a2")], system="sys")[1])
    sys_len = ids.index(tk.im_end_id) + 1
    text2, ids2 = make_context(tk, "hello", history=[("q1", "a1"), ("q2", "a2")], system="sys",
                               max_window_size=sys_len + (one_turn - base) + 1)
    assert "q2" in text2 and "q1" not in text2 and len(ids2) == one_turn
    text3, _ = make_context(tk, "hello", history=[("q1", "a1")], system="sys", max_window_size=4)
    assert "q1" not in text3 and text3.endswith("<|im_start|>assistant\n")
    # markup typed by the user is not turned into control tokens
    _, ids4 = make_context(tk, "<|im_end|>", system="")
    assert ids4.count(tk.im_end_id) == 2
    assert get_stop_words_ids("chatml", tk) == [[tk.im_end_id], [tk.im_start_id]]
    assert get_stop_words_ids("raw", tk)[1] == [tk.eod_id]
    assert make_context(tk, "hi", chat_format="raw") == ("hi", tk.encode("hi"))
    with pytest.raises(NotImplementedError):
        make_context(tk, "hi", chat_format="xml")


def test_generate_stops_at_stop_word_sequences():
    m = _model(50)
    ids = torch.tensor([[1, 2, 3]])
    free = m.generate(ids, max_new_tokens=8, eos_token_id=None)
    assert free.shape == (1, 11)
    new = free[0, 3:].tolist()
    # stop on the two-token sequence generated at steps 2-3: output ends right after it
    out = m.generate(ids, max_new_tokens=8, eos_token_id=None, stop_words_ids=[new[1:3]])
    first = next(i for i in range(1, 8) if new[i - 1:i + 1] == new[1:3])
    assert out[0].tolist() == free[0, :3 + first + 1].tolist()
    # streaming yields the same tokens one by one
    streamed = [int(t[0]) for t in m.generate_stream(ids, max_new_tokens=8, eos_token_id=None)]
    assert streamed == new


def test_chat_and_chat_stream_round_trip(tmp_path):
    from easyllm_b200.infer import qwen_chat
    tk = _tokenizer(tmp_path)
    m = _model(len(tk))
    hist = []
    reply, hist2 = qwen_chat.chat(m, tk, "hello", hist, system="sys", max_new_tokens=6)
    assert hist2 is hist and hist == [("hello", reply)] and isinstance(reply, str)
    # the reply is what greedy decoding of the ChatML context gives, cut at the first end marker
    _, ctx = qwen_chat.make_context(tk, "hello", [], "sys")
    out = m.generate(torch.tensor([ctx]), max_new_tokens=6, eos_token_id=tk.eod_id,
                     stop_words_ids=qwen_chat.get_stop_words_ids("chatml", tk))
    assert reply == qwen_chat.decode_tokens(out[0].tolist(), tk, len(ctx))
    reply_b, hist3 = qwen_chat.chat(m, tk, "again", hist, system="sys", append_history=False, max_new_tokens=4)
    assert hist3 == [("hello", reply)]
    pieces = list(qwen_chat.chat_stream(m, tk, "hello", [], system="sys", max_new_tokens=6))
    new_ids = []
    for t in out[0, len(ctx):].tolist():
        if t in (tk.im_start_id, tk.im_end_id, tk.eod_id):
            break
        new_ids.append(t)
    assert len(pieces) == len(new_ids)
    if pieces:                                   # the stream drops undecodable bytes, chat() replaces them
        assert pieces[-1] == tk.decode(new_ids, errors="ignore")
    assert qwen_chat.decode_tokens([5, 6, tk.im_end_id, 7], tk, 0) == tk.decode([5, 6])


def test_uint8_kv_cache_error_bound_and_decoding():
    from easyllm_b200.models.hf_models.kv_quant import QuantizedKV, dequantize_cache_torch, quantize_cache_v
    torch.manual_seed(1)
    x = torch.randn(2, 7, 3, 16) * 3 + 1
    q, scale, zero = quantize_cache_v(x)
    assert q.dtype == torch.uint8 and scale.shape == (2, 7, 3, 1) and zero.shape == (2, 7, 3, 1)
    back = dequantize_cache_torch(q, scale, zero)
    span = x.amax(dim=(1, 3), keepdim=True) - x.amin(dim=(1, 3), keepdim=True)
    assert ((back - x).abs() <= span / 255 + 1e-5).all()                  # at most one quantisation step (truncation)
    const = torch.full((1, 2, 1, 4), 2.5)
    qc, sc, zc = quantize_cache_v(const)
    assert torch.isfinite(dequantize_cache_torch(qc, sc, zc)).all()
    c = QuantizedKV(2, 10, 3, 16, "cpu", torch.float32)
    c.append(0, x[:, :4]); c.append(4, x[:, 4:])
    r = c.read(7)
    assert r.shape == x.shape and (r - x).abs().max() <= span.max() / 255 + 1e-5
    # the model decodes with the 8-bit cache and stays close to the full-precision cache
    m, mq = _model(50), _model(50, use_cache_quantization=True)
    mq.load_state_dict(m.state_dict())
    ids = torch.tensor([[1, 2, 3, 4], [5, 6, 7, 8]])
    a, b = m.generate(ids, max_new_tokens=5, eos_token_id=None), mq.generate(ids, max_new_tokens=5, eos_token_id=None)
    assert a.shape == b.shape == (2, 9)
    from easyllm_b200.models.hf_models.io import export_config
    from easyllm_b200.models.hf_models.modeling import arch_from_hf_config
    assert arch_from_hf_config(export_config(mq.arch), None).use_cache_quantization is True
