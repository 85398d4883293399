"""Family tokenizers registered in ``TOKENIZER_REGISTRY`` (the reference vendors them under
llm/models/hf_models/*/tokenization_*.py).

* ``SentencePieceTokenizer`` — loads a ``tokenizer.model`` (Baichuan, Baichuan2, InternLM,
  InternLM2 all ship one) and exposes the subset of the HF tokenizer API the parsers use.
* ``QWenTokenizer`` — byte-level BPE over a ``*.tiktoken`` rank file (base64 token, rank) with
  Qwen's pre-tokenisation regex and special tokens; implemented directly (no tiktoken dependency).
"""
from __future__ import annotations

import base64
import os

from ..config.registry import TOKENIZER_REGISTRY


class _Enc(dict):
    @property
    def input_ids(self):
        return self["input_ids"]


class SentencePieceTokenizer:
    vocab_files = ("tokenizer.model",)

    def __init__(self, vocab_file, bos_token="<s>", eos_token="</s>", unk_token="<unk>", pad_token=None,
                 add_bos_token=True, add_eos_token=False, **_):
        import sentencepiece as spm
        self.sp = spm.SentencePieceProcessor()
        self.sp.Load(vocab_file)
        self.vocab_file = vocab_file
        self.bos_token, self.eos_token, self.unk_token, self.pad_token = bos_token, eos_token, unk_token, pad_token
        self.add_bos_token, self.add_eos_token = add_bos_token, add_eos_token
        self.added = {}
        self.bos_token_id = self.sp.bos_id() if self.sp.bos_id() >= 0 else self.sp.PieceToId(bos_token)
        self.eos_token_id = self.sp.eos_id() if self.sp.eos_id() >= 0 else self.sp.PieceToId(eos_token)
        self.unk_token_id = self.sp.unk_id()
        self.pad_token_id = self.sp.PieceToId(pad_token) if pad_token else None

    @classmethod
    def from_pretrained(cls, path, **kw):
        f = path if os.path.isfile(path) else os.path.join(path, "tokenizer.model")
        return cls(f, **kw)

    @property
    def vocab_size(self):
        return self.sp.GetPieceSize()

    def __len__(self):
        return self.vocab_size + len(self.added)

    def add_special_tokens(self, mapping):
        n = 0
        for v in mapping.values():
            for t in (v if isinstance(v, (list, tuple)) else [v]):
                if t not in self.added and self.sp.PieceToId(t) == self.unk_token_id:
                    self.added[t] = self.vocab_size + len(self.added)
                    n += 1
        return n

    def encode(self, text, add_special_tokens=True):
        ids = []
        rest = text
        while self.added and rest:
            hit = min(((rest.find(t), t) for t in self.added if t in rest), default=None)
            if hit is None:
                break
            pos, t = hit
            ids += self.sp.EncodeAsIds(rest[:pos]) + [self.added[t]]
            rest = rest[pos + len(t):]
        ids += self.sp.EncodeAsIds(rest) if rest else []
        if add_special_tokens:
            ids = ([self.bos_token_id] if self.add_bos_token else []) + ids + ([self.eos_token_id] if self.add_eos_token else [])
        return ids

    def __call__(self, text, return_attention_mask=False, add_special_tokens=True, **_):
        ids = self.encode(text, add_special_tokens)
        out = _Enc(input_ids=ids)
        if return_attention_mask:
            out["attention_mask"] = [1] * len(ids)
        return out

    def decode(self, ids, skip_special_tokens=True, **_):
        ids = [int(ids)] if isinstance(ids, int) else [int(i) for i in ids]
        inv = {v: k for k, v in self.added.items()}
        special = {self.bos_token_id, self.eos_token_id, self.pad_token_id}
        out, buf = [], []
        for i in ids:
            if i in inv or i in special:
                if buf:
                    out.append(self.sp.DecodeIds(buf)); buf = []
                if not skip_special_tokens:
                    out.append(inv.get(i) or self.sp.IdToPiece(i))
            else:
                buf.append(i)
        if buf:
            out.append(self.sp.DecodeIds(buf))
        return "".join(out)

    def save_pretrained(self, path):
        import shutil
        os.makedirs(path, exist_ok=True)
        shutil.copy(self.vocab_file, os.path.join(path, "tokenizer.model"))


QWEN_PAT = r"""(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+"""
QWEN_SPECIAL = ["<|endoftext|>", "<|im_start|>", "<|im_end|>"] + [f"<|extra_{i}|>" for i in range(205)]


class QWenTokenizer:
    def __init__(self, vocab_file, extra_special=(), **_):
        import regex
        self.pat = regex.compile(QWEN_PAT)
        self.ranks = {}
        with open(vocab_file, "rb") as f:
            for line in f:
                if line.strip():
                    tok, rank = line.split()
                    self.ranks[base64.b64decode(tok)] = int(rank)
        self.decoder = {v: k for k, v in self.ranks.items()}
        self.special = {t: len(self.ranks) + i for i, t in enumerate(list(QWEN_SPECIAL) + list(extra_special))}
        self.special_inv = {v: k for k, v in self.special.items()}
        self.vocab_file = vocab_file
        self.eod_id = self.eos_token_id = self.special["<|endoftext|>"]
        self.im_start_id, self.im_end_id = self.special["<|im_start|>"], self.special["<|im_end|>"]
        self.eos_token, self.bos_token, self.pad_token = "<|endoftext|>", None, "<|endoftext|>"
        self.bos_token_id, self.pad_token_id = None, self.eod_id
        self._cache = {}

    @classmethod
    def from_pretrained(cls, path, **kw):
        f = path if os.path.isfile(path) else os.path.join(path, "qwen.tiktoken")
        return cls(f, **kw)

    @property
    def vocab_size(self):
        return len(self.ranks) + len(self.special)

    def __len__(self):
        return self.vocab_size

    def _bpe(self, piece: bytes):
        if piece in self._cache:
            return self._cache[piece]
        parts = [piece[i:i + 1] for i in range(len(piece))]
        while len(parts) > 1:
            best, at = None, -1
            for i in range(len(parts) - 1):
                r = self.ranks.get(parts[i] + parts[i + 1])
                if r is not None and (best is None or r < best):
                    best, at = r, i
            if best is None:
                break
            parts[at:at + 2] = [parts[at] + parts[at + 1]]
        ids = [self.ranks[p] for p in parts]
        self._cache[piece] = ids
        return ids

    def encode(self, text, add_special_tokens=True, allowed_special="all"):
        """``allowed_special``: "all", or the set of special-token strings that may be recognised in ``text``;
        markup outside that set is encoded as ordinary characters (an empty set for untrusted user text)."""
        allowed = self.special if allowed_special == "all" else [t for t in self.special if t in allowed_special]
        ids, rest = [], text
        while rest:
            hit = min(((rest.find(t), t) for t in allowed if t in rest), default=None)
            chunk, tok = (rest, None) if hit is None else (rest[:hit[0]], hit[1])
            for m in self.pat.findall(chunk):
                ids += self._bpe(m.encode("utf-8"))
            if tok is None:
                break
            ids.append(self.special[tok])
            rest = rest[len(chunk) + len(tok):]
        return ids

    def __call__(self, text, return_attention_mask=False, add_special_tokens=True, **_):
        ids = self.encode(text)
        out = _Enc(input_ids=ids)
        if return_attention_mask:
            out["attention_mask"] = [1] * len(ids)
        return out

    def decode(self, ids, skip_special_tokens=True, errors="replace", **_):
        ids = [int(ids)] if isinstance(ids, int) else [int(i) for i in ids]
        out, buf = [], b""
        for i in ids:
            if i in self.special_inv:
                out.append(buf.decode("utf-8", errors=errors)); buf = b""
                if not skip_special_tokens:
                    out.append(self.special_inv[i])
            else:
                buf += self.decoder[i]
        out.append(buf.decode("utf-8", errors=errors))
        return "".join(out)

    def add_special_tokens(self, mapping):
        return 0


class QWenVLTokenizer(QWenTokenizer):
    """Adds the image / box markup tokens and ``from_list_format`` of Qwen-VL."""
    VL = ("<img>", "</img>", "<imgpad>", "<ref>", "</ref>", "<box>", "</box>", "<quad>", "</quad>")

    def __init__(self, vocab_file, **kw):
        super().__init__(vocab_file, extra_special=self.VL, **kw)
        self.img_start_id, self.img_end_id, self.img_pad_id = (self.special[t] for t in self.VL[:3])

    @staticmethod
    def from_list_format(items):
        text, n = "", 0
        for it in items:
            if "image" in it:
                n += 1
                text += f"Picture {n}: <img>{it['image']}</img>\n"
            elif "text" in it:
                text += it["text"]
            elif "box" in it:
                text += (f"<ref>{it['ref']}</ref>" if "ref" in it else "") + \
                    "".join(f"<box>({b[0]},{b[1]}),({b[2]},{b[3]})</box>" for b in it["box"])
        return text


for _n in ("BaiChuanTokenizer", "BaiChuan2Tokenizer", "BaiChuan2Tokenizer13B", "InternLMTokenizer", "InternLM2Tokenizer"):
    TOKENIZER_REGISTRY.register(_n, SentencePieceTokenizer)
TOKENIZER_REGISTRY.register("QWenTokenizer", QWenTokenizer)
TOKENIZER_REGISTRY.register("QWenTokenizer_VL", QWenVLTokenizer)
