"""Family tokenizers: the byte-pair Qwen tokenizer on a synthetic rank file, Qwen-VL markup, registry names."""
import base64

import pytest


def _rank_file(path):
    # 256 single bytes, then merges in rank order: "he", "ll", "hell", "hello", " w", "or", " wor"
    toks = [bytes([i]) for i in range(256)] + [b"he", b"ll", b"hell", b"hello", b" w", b"or", b" wor"]
    with open(path, "wb") as f:
        for r, t in enumerate(toks):
            f.write(base64.b64encode(t) + b" " + str(r).encode() + b"\n")
    return toks


def test_qwen_bpe_merges_and_special_tokens(tmp_path):
    pytest.importorskip("regex")
    from easyllm_b200.data.tokenizers_hf import QWenTokenizer
    toks = _rank_file(tmp_path / "qwen.tiktoken")
    tk = QWenTokenizer.from_pretrained(str(tmp_path))
    ids = tk.encode("hello world")
    assert [toks[i] if i < len(toks) else None for i in ids] == [b"hello", b" wor", b"l", b"d"]
    assert tk.decode(ids) == "hello world"
    chat = "<|im_start|>user\nhello<|im_end|>"
    cid = tk.encode(chat)
    assert cid[0] == tk.im_start_id and cid[-1] == tk.im_end_id and tk.decode(cid, skip_special_tokens=False) == chat
    assert tk.decode(cid) == "user\nhello"
    assert len(tk) == len(toks) + len(tk.special) and tk.pad_token_id == tk.eod_id
    assert tk.decode(tk.encode("héllo ✓")) == "héllo ✓"                      # bytes outside the merges round-trip


def test_qwen_vl_list_format(tmp_path):
    pytest.importorskip("regex")
    from easyllm_b200.data.tokenizers_hf import QWenVLTokenizer
    _rank_file(tmp_path / "qwen.tiktoken")
    tk = QWenVLTokenizer.from_pretrained(str(tmp_path))
    text = tk.from_list_format([{"image": "a.jpg"}, {"text": "what is this?"}, {"ref": "dog", "box": [(1, 2, 3, 4)]}])
    assert text == "Picture 1: <img>a.jpg</img>\nwhat is this?<ref>dog</ref><box>(1,2),(3,4)</box>"
    ids = tk.encode(text)
    assert ids.count(tk.img_start_id) == 1 and ids.count(tk.img_end_id) == 1


def test_registry_has_the_reference_tokenizer_names():
    from easyllm_b200.config.registry import TOKENIZER_REGISTRY
    import easyllm_b200.data  # noqa: F401
    for name in ("LlamaTokenizer", "LlamaTokenizerFast", "AutoTokenizer", "QWenTokenizer", "SimpleTokenizer"):
        assert name in TOKENIZER_REGISTRY, name
