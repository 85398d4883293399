"""Qwen chat front end: ChatML context assembly, stop words, ``chat`` and ``chat_stream``.

Parity: llm/models/hf_models/qwen/qwen_generation_utils.py:109-201 (``get_stop_words_ids``, ``make_context``),
:261-300 (``decode_tokens``) and llm/models/hf_models/qwen/modeling_qwen.py:1182-1300 (``chat`` / ``chat_stream``
of ``QWenLMHeadModel``).  The functions take the model as an argument instead of being methods, so they work with
the generic ``CausalLM`` of ``models/hf_models/modeling.py`` for every family whose tokenizer has the ChatML ids.

Context layout (``chatml``)::

    <|im_start|>system\\n{system}<|im_end|>
    \\n<|im_start|>user\\n{q1}<|im_end|>\\n<|im_start|>assistant\\n{a1}<|im_end|>      (oldest kept turn first)
    ...
    \\n<|im_start|>user\\n{query}<|im_end|>\\n<|im_start|>assistant\\n

History turns are added newest-first while system + turns stay under ``max_window_size`` tokens; the first turn
that does not fit ends the walk (older ones are dropped even if shorter).
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch

History = List[Tuple[str, str]]
IM_START, IM_END = "<|im_start|>", "<|im_end|>"


def _plain(tokenizer, text):
    """Token ids of ``text`` with special-token markup inside it treated as ordinary characters."""
    try:
        return list(tokenizer.encode(text, allowed_special=set()))
    except TypeError:                       # tokenizers without the tiktoken-style argument
        return list(tokenizer.encode(text, add_special_tokens=False))


def get_stop_words_ids(chat_format: str, tokenizer) -> List[List[int]]:
    if chat_format == "raw":
        return [_plain(tokenizer, "Human:"), [tokenizer.eod_id]]
    if chat_format == "chatml":
        return [[tokenizer.im_end_id], [tokenizer.im_start_id]]
    raise NotImplementedError(f"Unknown chat format {chat_format!r}")


def make_context(tokenizer, query: str, history: Optional[History] = None, system: str = "",
                 max_window_size: int = 6144, chat_format: str = "chatml"):
    """Returns ``(raw_text, context_tokens)`` for one more user turn after ``history``."""
    history = history or []
    if chat_format == "raw":
        return query, _plain(tokenizer, query)
    if chat_format != "chatml":
        raise NotImplementedError(f"Unknown chat format {chat_format!r}")
    start, end, nl = [tokenizer.im_start_id], [tokenizer.im_end_id], _plain(tokenizer, "\n")

    def block(role, content):
        """One ``<|im_start|>role\\ncontent<|im_end|>`` block as (text, ids)."""
        ids = start + _plain(tokenizer, role) + nl + _plain(tokenizer, content) + end
        return f"{IM_START}{role}\n{content}{IM_END}", ids

    sys_text, sys_ids = block("system", system)
    kept_text, kept_ids = "", []
    for q, r in reversed(history):
        (qt, qi), (rt, ri) = block("user", q), block("assistant", r)
        turn_ids = nl + qi + nl + ri
        if len(sys_ids) + len(turn_ids) + len(kept_ids) >= max_window_size:
            break
        kept_ids = turn_ids + kept_ids
        kept_text = f"\n{qt}\n{rt}" + kept_text
    qt, qi = block("user", query)
    tokens = sys_ids + kept_ids + nl + qi + nl + start + _plain(tokenizer, "assistant") + nl
    text = sys_text + kept_text + f"\n{qt}\n{IM_START}assistant\n"
    return text, tokens


def decode_tokens(tokens: Sequence[int], tokenizer, context_length: int, chat_format: str = "chatml",
                  raw_text_len: int = 0, errors: str = "replace") -> str:
    """Text of the reply: the ids after the context up to the first end marker (``chatml``), or the decoded text
    after the prompt cut at ``Human:`` / ``<|endoftext|>`` (``raw``)."""
    tokens = [int(t) for t in tokens]
    if chat_format == "chatml":
        stop = {tokenizer.im_start_id, tokenizer.im_end_id}
        reply = []
        for t in tokens[context_length:]:
            if t in stop:
                break
            reply.append(t)
        return _decode(tokenizer, reply, errors).strip()
    if chat_format == "raw":
        text = _decode(tokenizer, tokens, errors)[raw_text_len:]
        for marker in ("Human:", "<|endoftext|>"):
            text = text.split(marker)[0]
        return text.strip()
    raise NotImplementedError(f"Unknown chat format {chat_format!r}")


def _decode(tokenizer, ids, errors):
    try:
        return tokenizer.decode(ids, errors=errors)
    except TypeError:
        return tokenizer.decode(ids)


def _device(model):
    return next(model.parameters()).device


def chat(model, tokenizer, query: str, history: Optional[History] = None, system: str = "You are a helpful assistant.",
         append_history: bool = True, stop_words_ids: Optional[List[List[int]]] = None, chat_format: str = "chatml",
         max_window_size: int = 6144, **gen_kwargs):
    """One chat turn: returns ``(response, history)``; ``history`` gains ``(query, response)`` unless told not to."""
    history = [] if history is None else history
    raw_text, ctx = make_context(tokenizer, query, history, system, max_window_size, chat_format)
    stops = list(stop_words_ids or []) + get_stop_words_ids(chat_format, tokenizer)
    ids = torch.tensor([ctx], dtype=torch.long, device=_device(model))
    gen_kwargs.setdefault("eos_token_id", tokenizer.eod_id)
    out = model.generate(ids, stop_words_ids=stops, **gen_kwargs)
    response = decode_tokens(out[0].tolist(), tokenizer, len(ctx), chat_format, len(raw_text))
    if append_history:
        history.append((query, response))
    return response, history


def chat_stream(model, tokenizer, query: str, history: Optional[History] = None,
                system: str = "You are a helpful assistant.", stop_words_ids: Optional[List[List[int]]] = None,
                chat_format: str = "chatml", max_window_size: int = 6144, **gen_kwargs):
    """Generator over the growing reply text, one item per decoded token (history is not modified)."""
    if chat_format != "chatml":
        raise NotImplementedError("chat_stream supports the chatml format only")
    raw_text, ctx = make_context(tokenizer, query, history or [], system, max_window_size, chat_format)
    stops = list(stop_words_ids or []) + get_stop_words_ids(chat_format, tokenizer)
    ids = torch.tensor([ctx], dtype=torch.long, device=_device(model))
    gen_kwargs.setdefault("eos_token_id", tokenizer.eod_id)
    got = []
    for tok in model.generate_stream(ids, stop_words_ids=stops, **gen_kwargs):
        got.append(int(tok[0]))
        if got[-1] in (tokenizer.im_start_id, tokenizer.im_end_id, tokenizer.eod_id):
            return
        yield _decode(tokenizer, got, "ignore")
