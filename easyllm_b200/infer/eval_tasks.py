"""Evaluation datasets and prompts: ``base`` (instruction/output json), C-Eval, CMMLU (5-shot from
the ``dev`` split), HumanEval (llm/utils/tools/dataset.py:220-422, prompt.py:9-119).

``build_eval_dataset`` yields ``{'tokens', 'meta'}`` items; ``text_postprocess`` extracts the
first capital letter for multiple choice or the function body for HumanEval; ``evaluate``
prints accuracy (and speculative-decoding acceptance statistics when present).
"""
from __future__ import annotations

import csv
import json
import os

from ..parallel.grid import get_grid
from ..utils.log import default_logger as logger

CHOICES = ("A", "B", "C", "D")


def filter_reply(text):
    text = text.split("\n\n")[0]
    if "```" in text:
        text = text.split("```")[1]
    if text.strip().startswith("def"):
        text = "\n".join(text.split("\n")[1:])
    if not text.startswith("    "):
        text = "    " + text.lstrip() if text.startswith(" ") else "\n".join("    " + ln for ln in text.split("\n"))
    return text


def first_capital_postprocess(text):
    return next((c for c in text if c.isupper()), "")


def text_postprocess(output, task_type):
    if task_type == "human_eval":
        return filter_reply(output)
    if task_type in ("cmmlu", "ceval"):
        return first_capital_postprocess(output)
    return output


def _read_csv(path):
    with open(path, newline="", encoding="utf-8") as f:
        return list(csv.DictReader(f))


def load_problems(task_type, question_dir, load_type="line", shots=5):
    """Returns (problems: {task_id: dict}, dev_prompts: {subject: few-shot prefix})."""
    problems, dev = {}, {}
    if task_type == "base":
        with open(question_dir) as f:
            metas = [json.loads(l) for l in f if l.strip()] if load_type == "line" else json.load(f)
        for i, d in enumerate(metas):
            problems[i] = {"task_id": i, "question": d.get("instruction", "") + d.get("input", ""), "answer": d.get("output", "")}
    elif task_type in ("cmmlu", "ceval"):
        test = os.path.join(question_dir, "test" if task_type == "cmmlu" else "val")
        qk, ak = ("Question", "Answer") if task_type == "cmmlu" else ("question", "answer")

        def subject(fn):
            base = fn.split(".")[0]
            return base if task_type == "cmmlu" else "_".join(base.split("_")[:-1])
        for fn in sorted(os.listdir(test)):
            for i, row in enumerate(_read_csv(os.path.join(test, fn))):
                tid = f"{subject(fn)}/{i}"
                problems[tid] = {"task_id": tid, "question": row[qk], **{c: row[c] for c in CHOICES}, "answer": row[ak]}
        devd = os.path.join(question_dir, "dev")
        for fn in sorted(os.listdir(devd)):
            rows = _read_csv(os.path.join(devd, fn))[:shots]
            name = subject(fn)
            dev[name] = "".join(
                f"题目：{r[qk]}\nA. {r['A']}\nB. {r['B']}\nC. {r['C']}\nD. {r['D']}\n答案是: {r[ak]}\n\n" for r in rows)
    elif task_type == "human_eval":
        with open(question_dir) as f:
            for l in f:
                if l.strip():
                    d = json.loads(l)
                    problems[d["task_id"]] = d
    else:
        raise ValueError(task_type)
    return problems, dev


def generate_prompt(problem, task_type, dev):
    if task_type == "human_eval":
        return problem["prompt"]
    if task_type == "base":
        return problem["question"]
    subj = str(problem["task_id"]).split("/")[0]
    q = problem
    lead = "以下是单项选择题，请直接给出正确答案的选项。\n" if task_type == "cmmlu" else "以下是单项选择题，请选出其中的正确答案。\n"
    return dev.get(subj, "") + lead + f"题目：{q['question']}\nA. {q['A']}\nB. {q['B']}\nC. {q['C']}\nD. {q['D']}\n答案是: "


class EvalDataset:
    def __init__(self, task_type, question_dir, tokenization=None, load_type="line"):
        self.task_type = task_type
        self.problems, self.dev = load_problems(task_type, question_dir, load_type)
        self.keys = list(self.problems)
        self.tokenization = tokenization

    def __len__(self):
        return len(self.keys)

    def __getitem__(self, i):
        p = self.problems[self.keys[i]]
        text = generate_prompt(p, self.task_type, self.dev)
        tokens = None
        if self.tokenization is not None:
            parser = self.tokenization.parser
            meta = parser.build_inference_meta(text, []) if hasattr(parser, "build_inference_meta") else {"text": text}
            tokens, _ = self.tokenization(meta)
        return {"tokens": tokens, "meta": {"task_id": p["task_id"], "input": text, "answer": p.get("answer", "")}}


def build_eval_dataset(task_type, question_dir, tokenization=None):
    return EvalDataset(task_type, question_dir, tokenization)


def save_results(path, samples):
    with open(path, "w") as f:
        for s in samples:
            f.write(json.dumps(s, ensure_ascii=False) + "\n")


def evaluate(task_type, samples):
    if task_type in ("cmmlu", "ceval"):
        ok = sum(text_postprocess(s["answer"] if "raw_output" not in s else s["raw_output"], task_type) == s.get("gold", s.get("answer"))
                 for s in samples)
        logger.info(f"Correct: {ok}; Ratio: {ok / max(1, len(samples)):.4f}")
        return ok / max(1, len(samples))
    steps = sum(s.get("infos", {}).get("count", 0) for s in samples)
    acc = sum(s.get("infos", {}).get("accept_length", 0) for s in samples)
    if steps:
        logger.info(f"Forward: {steps}; Accept_length: {acc}; Avg Accept_length: {acc / steps:.3f}")
    return None


def run_eval(runner, generator, generate_fn):
    """Eval mode of the megatron runner: shard problems over DP ranks, gather on rank 0."""
    from ..data.parsers import build_augmentation
    args, cfg = runner.args, runner.config
    icfg = cfg.get("infer_cfg", {})
    task = icfg.get("eval_task", getattr(args, "eval_task", "base"))
    tok = build_augmentation([cfg["infer_tokenization"]], runner.tokenizer).transforms[0]
    tok.parser.inference_mode = True
    ds = EvalDataset(task, icfg.get("question_file", getattr(args, "question_file", None)), tok)
    g = get_grid()
    out = []
    for i in range(g.dp_rank, len(ds), g.dp):
        item = ds[i]
        raw = generate_fn(args, item["tokens"], runner.engine, runner.tokenizer, args.force_eos_id, generator)
        out.append(dict(item["meta"], raw_output=raw, output=text_postprocess(raw, task), gold=item["meta"]["answer"]))
    if g.dp > 1:
        from ..parallel.hf_dist import all_gather_object
        out = [r for part in all_gather_object(out) for r in part]
    if g.rank == 0:
        save_results(icfg.get("result_file", getattr(args, "sample_file", "samples.jsonl")), out)
        if task in ("cmmlu", "ceval"):
            ok = sum(r["output"] == r["gold"] for r in out)
            logger.info(f"Correct: {ok}; Ratio: {ok / max(1, len(out)):.4f}")
    return out
