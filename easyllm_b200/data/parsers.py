"""Prompt parsers: raw records → ``{'input_ids', 'labels'}`` (registry ``PARSER_REGISTRY``).

Parity: llm/data/nlp_transforms.py:18-1094 — ``pretrain_bin``, ``tools``, ``intern_tools``,
``preprocess``, ``base`` (prompt types empty / llama / qwen / intern / baichuan2),
``general_chat``, ``combine_general_chat``, ``combine_dpo_general_chat``, ``simple_chat``,
``reward``, ``mini_rlhf``, ``QWen_Vl`` and the ``sense_tokenization`` augmentation wrapper.
All honour ``ignore_index`` (-100) for prompt tokens, ``keep_all_keys`` (train on every
token), ``only_last_answer``, ``drop_meta`` (drop over-long samples instead of truncating),
left-truncation to ``max_seq_length`` and ``inference_mode`` (returns ``(tokens, labels)``
lists without EOS).

Every chat-style parser is written on one primitive: a ``Segments`` builder collecting
``(text-or-token-ids, supervised?)`` pieces, so the prompt formats are declarative.
"""
from __future__ import annotations

import copy
import json

import numpy as np
import torch

from ..config.registry import AUGMENTATION_REGISTRY, PARSER_REGISTRY

IGNORE_INDEX = -100


class NLPCompose:
    def __init__(self, transforms):
        self.transforms = transforms

    def __call__(self, data):
        for t in self.transforms:
            data = t(data)
        return data


class Segments:
    """Token / label accumulator.  ``add(text, learn)`` tokenises without special tokens unless
    ``special=True`` (the first piece of a sample, which receives BOS)."""

    def __init__(self, tokenizer, ignore_index=IGNORE_INDEX):
        self.tok, self.ignore = tokenizer, ignore_index
        self.tokens, self.labels = [], []

    def ids(self, text, special=False):
        return list(self.tok(text, return_attention_mask=False, add_special_tokens=special)["input_ids"])

    def add(self, text, learn=False, special=False):
        return self.add_ids(self.ids(text, special), learn)

    def add_ids(self, ids, learn=False):
        ids = list(ids)
        self.tokens += ids
        self.labels += ids if learn else [self.ignore] * len(ids)
        return len(ids)

    def extend(self, other):
        self.tokens += other.tokens
        self.labels += other.labels

    def __len__(self):
        return len(self.tokens)


def _finish(tokens, labels, max_len, keep_all, drop_meta, keep="tail"):
    if drop_meta and len(tokens) > max_len:
        return None
    if keep == "tail":
        tokens, labels = tokens[-max_len:], labels[-max_len:]
    else:
        tokens, labels = tokens[:max_len], labels[:max_len]
    ids = torch.LongTensor(tokens)
    return {"input_ids": ids, "labels": ids.clone() if keep_all else torch.LongTensor(labels)}


class _ParserBase:
    def __init__(self, tokenizer, max_seq_length, ignore_index=IGNORE_INDEX, keep_all_keys=False,
                 inference_mode=False, drop_meta=False):
        self.tokenizer, self.max_seq_length, self.ignore_index = tokenizer, max_seq_length, ignore_index
        self.keep_all_keys, self.inference_mode, self.drop_meta = keep_all_keys, inference_mode, drop_meta

    def seg(self):
        return Segments(self.tokenizer, self.ignore_index)


@PARSER_REGISTRY.register("pretrain_bin")
class PretrainBinParser(_ParserBase):
    """Slice ``[start, end)`` of a token shard (.npy); documents end at EOS → ``cu_seqlens`` and
    per-document ``position_ids``; short slices are padded with ``len(tokenizer) − 1``."""

    def __init__(self, tokenizer, max_seq_length, **kw):
        super().__init__(tokenizer, max_seq_length, **kw)
        self.pad_token_id = len(tokenizer) - 1
        self._cache = {}

    def _shard(self, path):
        if path not in self._cache:
            if len(self._cache) > 8:
                self._cache.clear()
            self._cache[path] = np.load(path, mmap_mode="r")
        return self._cache[path]

    def get_cu_seqlens(self, tokens):
        ends = (np.where(np.asarray(tokens) == self.tokenizer.eos_token_id)[0] + 1).tolist()
        if not ends or ends[-1] != len(tokens):
            ends.append(len(tokens))
        return [0] + ends

    @staticmethod
    def get_position_ids(cu):
        return [p for a, b in zip(cu[:-1], cu[1:]) for p in range(b - a)]

    def __call__(self, meta):
        _, start, end = meta["bin_index"]
        tokens = np.asarray(self._shard(meta["path"])[start:end]).astype(np.int64)
        if len(tokens) < self.max_seq_length:
            tokens = np.concatenate((tokens, np.full(self.max_seq_length - len(tokens), self.pad_token_id, np.int64)))
        cu = self.get_cu_seqlens(tokens)
        ids = torch.from_numpy(tokens.copy())
        return {"input_ids": ids, "labels": ids.clone(), "cu_seqlens": torch.LongTensor(cu),
                "position_ids": torch.LongTensor(self.get_position_ids(cu))}


_PROMPTS = {
    "empty": "{q}",
    "llama": ("Below is an instruction that describes a task. Write a response that appropriately completes the "
              "request.\n\n### Instruction:\n\n{q}\n\n### Response:\n\n"),
    "qwen": "user\n{q}<|im_end|>\n<|im_start|>assistant\n",
    "intern": "<|User|>:{q}<eoh>\n<|Bot|>:",
}


@PARSER_REGISTRY.register("base")
class BaseParser(_ParserBase):
    def __init__(self, tokenizer, max_seq_length, split_paragraphs=False, ignore_index=IGNORE_INDEX,
                 keep_all_keys=False, inference_mode=False, prompt_type="empty", content_key="text", drop_meta=False):
        super().__init__(tokenizer, max_seq_length, ignore_index, keep_all_keys, inference_mode, drop_meta)
        if prompt_type not in ("empty", "llama", "qwen", "intern", "baichuan2"):
            raise ValueError(f"{prompt_type} has not supported.")
        self.prompt_type, self.content_key, self.split_paragraphs = prompt_type, content_key, split_paragraphs

    def build_input(self, text):
        if self.prompt_type == "baichuan2":
            return f"{self.tokenizer.decode(195)}{text}{self.tokenizer.decode(196)}"
        return _PROMPTS[self.prompt_type].format(q=text)

    def __call__(self, meta):
        if self.content_key not in meta:
            raise ValueError(f"content_key {self.content_key} not in meta keys ({list(meta.keys())})")
        text = self.build_input(meta[self.content_key])
        s = self.seg()
        if self.split_paragraphs:
            for i, para in enumerate(text.split("\n\n")):
                s.add(para + "\n\n", learn=True, special=(i == 0))
        else:
            s.add(text, learn=True, special=True)
        if self.inference_mode:
            return s.tokens, s.tokens
        s.add_ids([self.tokenizer.eos_token_id], learn=True)
        return _finish(s.tokens, s.labels, self.max_seq_length, True, self.drop_meta)


@PARSER_REGISTRY.register("preprocess")
class PreProcessParser(_ParserBase):
    def __call__(self, meta):
        s = self.seg()
        s.add(meta["inputs"], learn=self.keep_all_keys, special=True)
        s.add(meta.get("outputs", ""), learn=True)
        if self.inference_mode:
            return s.tokens, []
        s.add_ids([self.tokenizer.eos_token_id], learn=True)
        return _finish(s.tokens, s.labels, self.max_seq_length, False, self.drop_meta)


def _unpack_tool_meta(meta):
    if isinstance(meta, dict) and "input" in meta:
        inp = meta["input"]
        return inp.get("messages", []), inp.get("tools", []), inp.get("interpreter", [])
    if isinstance(meta, dict) and "messages" in meta:
        return meta["messages"], meta.get("tools", []), meta.get("interpreter", [])
    return meta, [], []


@PARSER_REGISTRY.register("tools")
class ToolParser(_ParserBase):
    def __init__(self, tokenizer, max_seq_length, ignore_index=IGNORE_INDEX, keep_all_keys=False,
                 inference_mode=False, drop_meta=False, prompt_template=None, use_system=True, use_knowledge=True,
                 ensure_ascii=False):
        super().__init__(tokenizer, max_seq_length, ignore_index, keep_all_keys, inference_mode, drop_meta)
        t = prompt_template or {}
        self.system_prompt = t.get("sytem_prompt", t.get("system_prompt", "<system>: "))
        self.user_prompt = t.get("user_prompt", "<user>: ")
        self.assistant_prompt = t.get("assistant_prompt", "<assistant>: ")
        self.tool_calls_start = t.get("tool_calls_start", "<tool_calls_start>\n")
        self.tool_calls_end = t.get("tool_calls_end", "<tool_calls_end>\n")
        self.tool_response_prompt = t.get("tool_response_prompt", "<tool_response>:\n")
        self.tool_define = t.get("tool_define", "<tools_define>:\n")
        self.knowledge_prompt = t.get("knowledge_prompt", "<knowledge>: ")
        self.use_system, self.use_knowledge, self.ensure_ascii = use_system, use_knowledge, ensure_ascii

    def __call__(self, meta):
        messages, tools, _ = _unpack_tool_meta(meta)
        s = self.seg()
        head = (self.tool_define if tools else "") + "".join(
            json.dumps(t["function"], ensure_ascii=self.ensure_ascii) + "\n" for t in tools)
        s.add(head, special=True)
        for m in messages:
            role, content = m["role"], m.get("content")
            if role == "system" and self.use_system and content != "":
                s.add(f"{self.system_prompt}{content}\n")
            elif role == "user":
                s.add(f"{self.user_prompt}{content}\n")
            elif role == "knowledge" and self.use_knowledge:
                s.add(f"{self.knowledge_prompt}{content}\n")
            elif role == "assistant":
                s.add(self.assistant_prompt)
                text = content or ""
                if m.get("tool_calls"):
                    text += self.tool_calls_start + "".join(
                        json.dumps(c["function"], ensure_ascii=self.ensure_ascii) + "\n" for c in m["tool_calls"])
                    text += self.tool_calls_end
                s.add(text, learn=True)
                if not self.inference_mode:
                    s.add_ids([self.tokenizer.eos_token_id], learn=True)
            elif role == "tool":
                s.add(f"{self.tool_response_prompt}{content}")
        if self.inference_mode:
            s.add(self.assistant_prompt)
            return s.tokens, []
        return _finish(s.tokens, s.labels, self.max_seq_length, self.keep_all_keys, self.drop_meta)


@PARSER_REGISTRY.register("intern_tools")
class InternToolParser(_ParserBase):
    def __init__(self, tokenizer, max_seq_length, ignore_index=IGNORE_INDEX, keep_all_keys=False,
                 inference_mode=False, drop_meta=False, prompt_template=None, use_system=True, use_knowledge=False,
                 use_interpreter=True, ensure_ascii=False, tool_mode="merge"):
        super().__init__(tokenizer, max_seq_length, ignore_index, keep_all_keys, inference_mode, drop_meta)
        t = prompt_template or {}
        self.cs, self.ce = t.get("conversation_start", "<|im_start|>"), t.get("conversation_end", "<|im_end|>")
        self.action_start, self.action_end = t.get("action_start", "<|action_start|>"), t.get("action_end", "<|action_end|>")
        self.plugin, self.interp = t.get("plugin", "<|plugin|>"), t.get("interpreter", "<|interpreter|>")
        self.use_system, self.use_knowledge, self.use_interpreter = use_system, use_knowledge, use_interpreter
        self.ensure_ascii, self.tool_mode = ensure_ascii, tool_mode
        if use_knowledge:
            raise NotImplementedError("intern_tools has no knowledge role")

    def __call__(self, meta):
        messages, tools, interpreter = _unpack_tool_meta(meta)
        s = self.seg()
        s.add_ids([self.tokenizer.bos_token_id])
        conv = messages
        if self.use_system and messages and messages[0]["role"] == "system" and messages[0]["content"] != "":
            s.add(f"{self.cs}system\n{messages[0]['content']}{self.ce}\n")
            conv = messages[1:]
        if self.use_interpreter and interpreter:
            if len(interpreter) != 1 or interpreter[0]["name"] != "python_interpreter":
                raise ValueError("Only support python interpreter now!")
            s.add(f"{self.cs}system name={self.interp}\n{interpreter[0]['description']}\n{self.ce}\n")
        plug = [copy.deepcopy(t["function"]) for t in tools
                if not (self.use_interpreter and t["function"]["name"] == "python_interpreter")]
        if plug:
            body = json.dumps(plug, ensure_ascii=self.ensure_ascii) if self.tool_mode == "merge" else \
                "\n".join(json.dumps(t, ensure_ascii=self.ensure_ascii) for t in plug)
            s.add(f"{self.cs}system name={self.plugin}\n{body}\n{self.ce}\n")
        for m in conv:
            role = m["role"]
            if role == "user":
                s.add(f"{self.cs}user\n{m['content']}{self.ce}\n")
            elif role == "assistant":
                s.add(f"{self.cs}assistant\n")
                text = m.get("content") or ""
                if m.get("tool_calls"):
                    text += self.action_start
                    for c in m["tool_calls"]:
                        fn = c["function"]
                        if self.use_interpreter and fn.get("name") == "python_interpreter":
                            text += f"{self.interp}\n{fn['arguments']['code']}\n"
                        else:
                            text += f"{self.plugin}\n{json.dumps(fn, ensure_ascii=self.ensure_ascii)}\n"
                    text += self.action_end
                if not self.inference_mode:
                    text += f"{self.ce}\n"
                s.add(text, learn=True)
            elif role == "tool":
                tag = self.interp if (self.use_interpreter and m.get("name") == "python_interpreter") else self.plugin
                s.add(f"{self.cs}environment name={tag}\n{m['content']}{self.ce}\n")
        if self.inference_mode:
            s.add(f"{self.cs}assistant\n")
            return s.tokens, []
        return _finish(s.tokens, s.labels, self.max_seq_length, self.keep_all_keys, self.drop_meta)


class _ChatBase(_ParserBase):
    """Shared record handling of the chat parsers: alpaca-style dicts, ``{'messages': …}``
    dicts and plain role/content lists → (system text, history, question, answer)."""

    def convert2chat(self, meta):
        out = [{"role": "system", "content": meta["system"]}] if "system" in meta else []
        out.append({"role": "user", "content": meta.get("instruction", "") + meta.get("input", "")})
        out.append({"role": "assistant", "content": meta.get("output", "")})
        return out

    def split_dialog(self, meta, system):
        if isinstance(meta, dict):
            if "messages" in meta:
                system += meta.get("system", "")
                meta = meta["messages"]
            if "input" in meta:
                meta = self.convert2chat(meta)
        question = answer = ""
        history = []
        if len(meta) <= 1:
            for it in meta:
                if it["role"] == "user":
                    question += it.get("content", "")
                if it["role"] == "assistant":
                    answer += it.get("content", "")
        elif self.inference_mode:
            question, history = meta[-1]["content"], meta[:-1]
        else:
            answer, question, history = meta[-1]["content"], meta[-2]["content"], meta[:-2]
        return system, history, question, answer

    def build_inference_meta(self, text, history=None):
        return list(history or []) + [{"role": "user", "content": text}]

    def __call__(self, meta):
        tokens, labels = self.get_tokens_labels(meta)
        if self.inference_mode:
            return tokens, labels
        if tokens is None:
            return None
        ids = torch.LongTensor(tokens)
        return {"input_ids": ids, "labels": ids.clone() if self.keep_all_keys else torch.LongTensor(labels)}

    def assemble(self, head, hist, tail, budget_slack=0):
        """head + history + tail with history clipped from the oldest side when too long, then the
        whole sample cut on the right; ``only_last_answer`` masks everything before ``answer``."""
        n = len(head) + len(hist) + sum(len(t) for t in tail)
        if n > self.max_seq_length:
            if self.drop_meta:
                return None, None
            cut = n - (self.max_seq_length + budget_slack)
            hist.tokens, hist.labels = hist.tokens[cut:], hist.labels[cut:]
        parts = [head, hist] + tail
        tokens = [t for p in parts for t in p.tokens]
        labels = [t for p in parts for t in p.labels]
        if self.only_last_answer:
            k = len(tokens) - len(tail[-1])
            labels = [self.ignore_index] * k + labels[k:]
        return tokens[:self.max_seq_length], labels[:self.max_seq_length]


@PARSER_REGISTRY.register("general_chat")
class GeneralChatParser(_ChatBase):
    def __init__(self, tokenizer, max_seq_length, ignore_index=IGNORE_INDEX, keep_all_keys=False,
                 only_last_answer=False, prompt_template=None, inference_mode=False, drop_meta=False):
        super().__init__(tokenizer, max_seq_length, ignore_index, keep_all_keys, inference_mode, drop_meta)
        t = prompt_template or {}
        self.only_last_answer = only_last_answer
        self.system_prompt = t.get("system_prompt", "<系统> ") + t.get("predefine_prompt", "")
        self.dialog_history_prompt = t.get("dialog_history_prompt", "<对话历史> ")
        self.question_prompt = t.get("question_prompt", "<最新问题> ")
        self.knowledge_prompt = t.get("knowledge_prompt", "<知识> ")
        self.answer_prompt = t.get("answer_prompt", "SenseChat:")
        self.user_prompt = t.get("user_prompt", "用户:")

    def get_tokens_labels(self, meta):
        system, dialog, question, answer = self.split_dialog(meta, self.system_prompt)
        knowledge = self.knowledge_prompt
        for it in dialog:
            if it["role"] == "system":
                system += it["content"]
            if it["role"] == "knowledge":
                knowledge += it["content"]
        turns = [it for it in dialog if it["role"] in ("user", "assistant")]
        head = self.seg(); head.add(system, special=True)
        hist = self.seg()
        eos = self.tokenizer.eos_token_id
        for i, it in enumerate(turns):
            lead = self.dialog_history_prompt if i == 0 else ""
            if it["role"] == "user":
                hist.add(f"{lead}{self.user_prompt}{it['content']}")
            else:
                hist.add(f"{lead}{self.answer_prompt}")
                ids = hist.ids(it["content"])
                # an answer that opens the history is context only, but its EOS is still supervised
                hist.add_ids(ids, learn=(i != 0))
                hist.add_ids([eos], learn=True)
        know = self.seg(); know.add(knowledge)
        ques = self.seg(); ques.add(f"{self.question_prompt}{self.user_prompt}{question}")
        ans = self.seg(); ans.add(self.answer_prompt)
        ans.add_ids(ans.ids(answer) + ([] if self.inference_mode else [eos]), learn=True)
        return self.assemble(head, hist, [know, ques, ans])


@PARSER_REGISTRY.register("combine_general_chat")
class CombinedGeneralChatParser(GeneralChatParser):
    """Per-record override: ``{'keep_all_keys': True, 'convs': […]}`` / ``{'only_last_answer': True, …}``."""

    def __init__(self, tokenizer, max_seq_length, **kw):
        super().__init__(tokenizer, max_seq_length, **kw)
        k = dict(kw); k["only_last_answer"] = True
        self.last_answer_parser = GeneralChatParser(tokenizer, max_seq_length, **k)
        k.update(only_last_answer=False, keep_all_keys=True)
        self.keep_all_parser = GeneralChatParser(tokenizer, max_seq_length, **k)

    def __call__(self, meta):
        if isinstance(meta, dict) and meta.get("keep_all_keys", False):
            return self.keep_all_parser(meta["convs"])
        if isinstance(meta, dict) and meta.get("only_last_answer", False):
            return self.last_answer_parser(meta["convs"])
        return GeneralChatParser.__call__(self, meta)


@PARSER_REGISTRY.register("combine_dpo_general_chat")
class CombinedDPOSFTParser(CombinedGeneralChatParser):
    """Preference pairs ``yw`` / ``yl`` with offline reference log-probs; a record whose
    ``yw_logp`` is a single value ≥ 1 is plain SFT data (scores 999999 switch the loss to SFT)."""

    def __init__(self, tokenizer, max_seq_length, inference_mode=False, average_log_prob=False, **kw):
        if inference_mode:
            raise ValueError("dpo_rlhf parser does not support model inference")
        self.average_log_prob = average_log_prob
        super().__init__(tokenizer, max_seq_length, **kw)

    def _pair(self, yw, yl, scores):
        return {"input_ids": [yw["input_ids"], yl["input_ids"]], "labels": [yw["labels"], yl["labels"]],
                "scores": torch.FloatTensor(scores)}

    def __call__(self, meta):
        parent = CombinedGeneralChatParser.__call__
        logp_w = torch.FloatTensor(meta["yw_logp"])
        if len(logp_w) == 1 and logp_w[0] >= 1:
            return self._pair(parent(self, meta["yw"]), parent(self, meta["yl"]), [999999, 999999])
        yw = parent(self, {"convs": meta["yw"], "only_last_answer": True})
        yl = parent(self, {"convs": meta["yl"], "only_last_answer": True})
        scores = []
        for res, lp in ((yw, logp_w), (yl, torch.FloatTensor(meta["yl_logp"]))):
            m = (res["labels"] != self.ignore_index)[1:].float()     # log-probs start at the second token
            sc = (lp * m).sum(-1)
            scores.append(float(sc / m.sum(-1)) if self.average_log_prob else float(sc))
        return self._pair(yw, yl, scores)


@PARSER_REGISTRY.register("simple_chat")
class SimpleChatParser(_ChatBase):
    def __init__(self, tokenizer, max_seq_length, ignore_index=IGNORE_INDEX, keep_all_keys=False,
                 only_last_answer=False, prompt_template=None, inference_mode=False, drop_meta=False):
        super().__init__(tokenizer, max_seq_length, ignore_index, keep_all_keys, inference_mode, drop_meta)
        t = prompt_template or {}
        self.only_last_answer = only_last_answer
        self.system_prompt = t.get("system_prompt", "<|System>|>:") + t.get("predefine_prompt", "")
        self.question_prompt = t.get("qustion_prompt", t.get("question_prompt", "<|Human|>:"))
        self.answer_prompt = t.get("answer_prompt", "<|Assistant|>:")
        self.eoh, self.eosys, self.eoa = t.get("eoh", "\n"), t.get("eosys", "\n"), t.get("eoa", "")

    # hooks the multimodal subclass overrides
    def system_segment(self, system):
        s = self.seg(); s.add(system, special=True); return s

    def question_segment(self, question):
        s = self.seg(); s.add(f"{self.question_prompt}{question}{self.eoh}"); return s

    def answer_segment(self, answer):
        s = self.seg(); s.add(self.answer_prompt)
        if self.inference_mode:
            s.add(answer, learn=True)
        else:
            s.add_ids(s.ids(answer + self.eoa) + [self.tokenizer.eos_token_id], learn=True)
        return s

    def history_segment(self, turns):
        h = self.seg()
        for i, it in enumerate(turns):
            if it["role"] == "user":
                h.add(f"{self.question_prompt}{it['content']}{self.eoh}")
            else:
                h.add(self.answer_prompt)
                h.add_ids(h.ids(f"{it['content']}{self.eoa}") + [self.tokenizer.eos_token_id], learn=(i != 0))
        return h

    def get_tokens_labels(self, meta):
        system, dialog, question, answer = self.split_dialog(meta, self.system_prompt)
        for it in dialog:
            if it["role"] == "system":
                system += it["content"]
        system = f"{system}{self.eosys}"
        turns = [it for it in dialog if it["role"] in ("user", "assistant")]
        return self.assemble(self.system_segment(system), self.history_segment(turns),
                             [self.question_segment(question), self.answer_segment(answer)])


@PARSER_REGISTRY.register("reward")
class RewardParser(_ParserBase):
    def __init__(self, tokenizer, max_seq_length, ignore_index=IGNORE_INDEX, keep_all_keys=False,
                 return_type="token_ids", inference_mode=False):
        super().__init__(tokenizer, max_seq_length, ignore_index, keep_all_keys, inference_mode)

    def __call__(self, meta):
        s = self.seg()
        q = s.ids(meta["input_text"], special=True)
        good = s.ids(meta["choice"])
        eos = [self.tokenizer.eos_token_id]
        if not self.inference_mode:
            bad = s.ids(meta.get("bad_answer", ""))
            return {"input_ids": (torch.LongTensor((q + good + eos)[:self.max_seq_length]),
                                  torch.LongTensor((q + bad + eos)[:self.max_seq_length]))}
        over = len(q) + len(good) - self.max_seq_length
        if over > 0:
            q = q[over:]
        return {"input_ids": torch.LongTensor(q + good),
                "labels": torch.LongTensor([self.ignore_index] * len(q) + good)[:self.max_seq_length]}


@PARSER_REGISTRY.register("mini_rlhf")
class MiniRLHFParser(_ParserBase):
    def __init__(self, tokenizer, max_seq_length, ignore_index=IGNORE_INDEX, keep_all_keys=False,
                 return_type="token_ids", inference_mode=False):
        super().__init__(tokenizer, max_seq_length, ignore_index, keep_all_keys, inference_mode)

    def __call__(self, meta):
        if self.inference_mode:
            return meta["question"]
        if not self.tokenizer.eos_token:
            raise ValueError("the tokenizer must have an eos_token")
        s = self.seg()
        q = s.ids(meta["question"], special=True)
        ids, labels = [], []
        for ans in meta["answers"]:
            a = s.ids(f"{ans}{self.tokenizer.eos_token}")
            ids.append(torch.LongTensor(q + a)[-self.max_seq_length:])
            labels.append(torch.LongTensor([self.ignore_index] * len(q) + a)[-self.max_seq_length:])
        return {"input_ids": ids, "labels": labels, "scores": torch.FloatTensor(meta["scores"])}


@PARSER_REGISTRY.register("QWen_Vl")
class QWenVLParser(SimpleChatParser):
    """ChatML framing for Qwen-VL: every turn is ``<|im_start|>role\\n…<|im_end|>\\n``; the frame
    tokens (im_start / im_end / newline) are supervised, the role name and user text are not."""

    def __init__(self, tokenizer, max_seq_length, ignore_index=IGNORE_INDEX, prompt_template=None,
                 inference_mode=False, only_last_answer=False, keep_all_keys=False, drop_meta=False):
        super().__init__(tokenizer, max_seq_length, ignore_index, keep_all_keys, only_last_answer,
                         prompt_template, inference_mode, drop_meta)
        t = prompt_template or {}
        self.system_prompt = t.get("system_prompt", "You are a helpful assistant.")
        self.question_prompt = t.get("qustion_prompt", t.get("question_prompt", "<|im_start|>user\n"))
        self.answer_prompt = t.get("answer_prompt", "<|im_start|>assistant\n")
        self.eoh = t.get("eoh", "<|im_end|>\n")
        self.eosys = t.get("eosys", "<|im_end|>\n")
        self.nl = list(tokenizer("\n")["input_ids"])
        self.im_start, self.im_end = tokenizer.im_start_id, tokenizer.im_end_id

    def _framed(self, ids, learn_body_from=None):
        """ids = [im_start, …, im_end, nl]: supervise the frame; the body from ``learn_body_from`` on."""
        s = self.seg()
        body_lab = [self.ignore_index] * (len(ids) - 3)
        if learn_body_from is not None:
            body = ids[1:-2]
            body_lab = [self.ignore_index] * learn_body_from + body[learn_body_from:]
        s.tokens = list(ids)
        s.labels = [self.im_start] + body_lab + [self.im_end] + self.nl
        return s

    def system_segment(self, system):
        return self._framed(self.seg().ids("<|im_start|>system\n" + system, special=True))

    def question_segment(self, question):
        return self._framed(self.seg().ids(f"{self.question_prompt}{question}{self.eoh}"))

    def _assistant(self, content, learn):
        head = self.seg().ids("<|im_start|>assistant")
        ids = head + self.nl + self.seg().ids(content) + [self.im_end] + self.nl
        s = self._framed(ids, learn_body_from=len(head) - 1 + len(self.nl))
        if not learn:
            s.labels = [self.ignore_index] * len(s.labels)
        return s

    def history_segment(self, turns):
        h = self.seg()
        for i, it in enumerate(turns):
            if it["role"] == "user":
                ids = self.seg().ids("<|im_start|>user") + self.nl + self.seg().ids(it["content"]) + [self.im_end] + self.nl
                h.extend(self._framed(ids))
            else:
                h.extend(self._assistant(it["content"], learn=(i != 0)))
        return h

    def answer_segment(self, answer):
        if self.inference_mode:
            s = self.seg(); s.add(self.answer_prompt); s.add(answer, learn=True); return s
        return self._assistant(answer + self.eoa, learn=True)


def build_parser(parser_type, parser_kwargs):
    return PARSER_REGISTRY.build({"type": parser_type, "kwargs": parser_kwargs})


@AUGMENTATION_REGISTRY.register("sense_tokenization")
class SenseTokenization:
    def __init__(self, tokenizer, max_seq_length, parser_type=None, parser_kwargs=None, ignore_index=IGNORE_INDEX,
                 with_tokenizer=True):
        kw = dict(parser_kwargs or {})
        kw.update(tokenizer=tokenizer, max_seq_length=max_seq_length, ignore_index=ignore_index)
        if parser_type in (None, "default"):
            parser_type = "base"
        elif parser_type in ("chat", "sense_chat"):
            parser_type = "general_chat"
        self.parser = build_parser(parser_type, kw)

    def __call__(self, *a, **k):
        return self.parser(*a, **k)


def build_transformer(cfg_list, tokenizer):
    """``transformer: [ {type, kwargs}, … ]`` of a dataset config → composed callable."""
    ts = []
    for c in cfg_list or []:
        c = {"type": c["type"], "kwargs": dict(c.get("kwargs") or {})}
        c["kwargs"].pop("with_tokenizer", None)
        c["kwargs"]["tokenizer"] = tokenizer
        ts.append(AUGMENTATION_REGISTRY.build(c))
    return NLPCompose(ts)


build_augmentation = build_transformer
