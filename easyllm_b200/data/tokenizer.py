"""Tokenizer construction (llm/data/tokenizer.py:9-42).

``build_tokenizer(cfg)`` resolves ``cfg.type`` in ``TOKENIZER_REGISTRY`` and calls
``from_pretrained(tokenizer_name_or_path, **kwargs)``; ``special_tokens`` are added, and
``padded_vocab_size = pad_vocab_size_to`` or the vocabulary size rounded up to
``make_vocab_size_divisible_by`` (× TP so vocab-parallel shards stay equal).
``SimpleTokenizer`` is a dependency-free byte-level tokenizer for tests and synthetic runs.
"""
from __future__ import annotations

from ..config.registry import TOKENIZER_REGISTRY
from ..utils.log import default_logger as logger


class SimpleTokenizer:
    """Byte-level tokenizer: ids 0..255 are bytes, then <s>=256, </s>=257, <unk>=258, <pad>."""

    def __init__(self, vocab_size=32000, **kw):
        self._vocab = max(vocab_size, 260)
        self.bos_token, self.eos_token, self.unk_token, self.pad_token = "<s>", "</s>", "<unk>", "<pad>"
        self.bos_token_id, self.eos_token_id, self.unk_token_id = 256, 257, 258
        self.pad_token_id = self._vocab - 1
        self.vocab_size = self._vocab
        self._special = {self.bos_token: 256, self.eos_token: 257, self.unk_token: 258}

    @classmethod
    def from_pretrained(cls, tokenizer_name_or_path=None, **kw):
        return cls(**{k: v for k, v in kw.items() if k == "vocab_size"})

    def __len__(self):
        return self._vocab

    def encode(self, text, add_special_tokens=True):
        ids = []
        i = 0
        while i < len(text):
            hit = next((t for t in self._special if text.startswith(t, i)), None)
            if hit:
                ids.append(self._special[hit]); i += len(hit)
            else:
                ids.extend(text[i].encode("utf-8")); i += 1
        return ([self.bos_token_id] if add_special_tokens else []) + ids

    def __call__(self, text, return_attention_mask=False, add_special_tokens=True, **kw):
        ids = self.encode(text, add_special_tokens)

        class _Enc(dict):
            input_ids = ids
        out = _Enc(input_ids=ids)
        if return_attention_mask:
            out["attention_mask"] = [1] * len(ids)
        return out

    def decode(self, ids, skip_special_tokens=True, **kw):
        if isinstance(ids, int):
            ids = [ids]
        inv = {v: k for k, v in self._special.items()}
        out, buf = [], bytearray()
        for t in (int(x) for x in ids):
            if t < 256:
                buf.append(t)
                continue
            if buf:
                out.append(buf.decode("utf-8", errors="replace")); buf = bytearray()
            if not skip_special_tokens and t in inv:
                out.append(inv[t])
        if buf:
            out.append(buf.decode("utf-8", errors="replace"))
        return "".join(out)

    def add_special_tokens(self, mapping):
        return 0

    def save_pretrained(self, path):
        import json, os
        os.makedirs(path, exist_ok=True)
        with open(os.path.join(path, "simple_tokenizer.json"), "w") as f:
            json.dump({"vocab_size": self._vocab}, f)


TOKENIZER_REGISTRY.register("SimpleTokenizer", SimpleTokenizer)


def _register_hf():
    try:
        from transformers import AutoTokenizer, LlamaTokenizer, LlamaTokenizerFast
    except Exception:
        return
    for name, cls in (("AutoTokenizer", AutoTokenizer), ("LlamaTokenizer", LlamaTokenizer),
                      ("LlamaTokenizerFast", LlamaTokenizerFast)):
        if name not in TOKENIZER_REGISTRY:
            TOKENIZER_REGISTRY.register(name, cls)


_register_hf()


def build_tokenizer(cfg_tokenizer, tp_size=1):
    cfg = dict(cfg_tokenizer)
    kw = dict(cfg.get("kwargs") or {})
    path = kw.pop("tokenizer_name_or_path", None)
    cls = TOKENIZER_REGISTRY.get(cfg["type"])
    tok = cls.from_pretrained(path, **kw) if path is not None else cls.from_pretrained(**kw)
    special = cfg.get("special_tokens")
    if special:
        tok.add_special_tokens(special)
    if getattr(tok, "pad_token", None) is None and getattr(tok, "eos_token", None) is not None:
        try:
            tok.pad_token = tok.eos_token
        except Exception:
            pass
    pad_to = cfg.get("pad_vocab_size_to")
    if pad_to is not None:
        if pad_to < len(tok):
            raise ValueError(f"pad_vocab_size_to ({pad_to}) is smaller than the vocabulary ({len(tok)})")
        tok.padded_vocab_size = pad_to
    else:
        mult = cfg.get("make_vocab_size_divisible_by", 1) * max(1, tp_size)
        tok.padded_vocab_size = (len(tok) + mult - 1) // mult * mult
    logger.info(f"tokenizer {cfg['type']}: vocab {len(tok)}, padded to {tok.padded_vocab_size}")
    return tok
