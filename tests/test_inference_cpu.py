"""Evaluation datasets / prompts / post-processing and the interactive generation loop, on CPU."""
import csv
import json
import os
import types

import torch


def _write_csv(path, rows, header):
    os.makedirs(os.path.dirname(path), exist_ok=True)
    with open(path, "w", newline="", encoding="utf-8") as f:
        w = csv.DictWriter(f, fieldnames=header)
        w.writeheader()
        for r in rows:
            w.writerow(r)


def test_ceval_prompts_and_scoring(tmp_path):
    from easyllm_b200.infer import eval_tasks as et
    header = ["id", "question", "A", "B", "C", "D", "answer"]
    dev = [{"id": i, "question": f"dev q{i}", "A": "1", "B": "2", "C": "3", "D": "4", "answer": "B"} for i in range(6)]
    val = [{"id": i, "question": f"val q{i}", "A": "a", "B": "b", "C": "c", "D": "d", "answer": "ACD"[i]} for i in range(3)]
    _write_csv(str(tmp_path / "dev" / "college_physics_dev.csv"), dev, header)
    _write_csv(str(tmp_path / "val" / "college_physics_val.csv"), val, header)
    ds = et.build_eval_dataset("ceval", str(tmp_path))
    assert len(ds) == 3
    item = ds[1]
    assert item["meta"]["task_id"] == "college_physics/1" and item["meta"]["answer"] == "C"
    prompt = item["meta"]["input"]
    assert prompt.count("答案是") == 6 and "dev q4" in prompt and "dev q5" not in prompt   # five shots + the question
    assert prompt.rstrip().endswith("答案是:")
    samples = [{"raw_output": " the answer is C because", "gold": "C"}, {"raw_output": "b", "gold": "B"}]
    assert et.text_postprocess(samples[0]["raw_output"], "ceval") == "C"
    assert abs(et.evaluate("ceval", samples) - 0.5) < 1e-9


def test_cmmlu_and_base_and_humaneval(tmp_path):
    from easyllm_b200.infer import eval_tasks as et
    header = ["Question", "A", "B", "C", "D", "Answer"]
    rows = [{"Question": f"q{i}", "A": "1", "B": "2", "C": "3", "D": "4", "Answer": "D"} for i in range(2)]
    _write_csv(str(tmp_path / "cm" / "dev" / "anatomy.csv"), rows, header)
    _write_csv(str(tmp_path / "cm" / "test" / "anatomy.csv"), rows, header)
    ds = et.build_eval_dataset("cmmlu", str(tmp_path / "cm"))
    assert ds[0]["meta"]["task_id"] == "anatomy/0" and "请直接给出正确答案的选项" in ds[0]["meta"]["input"]
    base = tmp_path / "base.jsonl"
    base.write_text(json.dumps({"instruction": "Add ", "input": "1+1", "output": "2"}) + "\n")
    b = et.build_eval_dataset("base", str(base))
    assert b[0]["meta"]["input"] == "Add 1+1" and b[0]["meta"]["answer"] == "2"
    he = tmp_path / "he.jsonl"
    he.write_text(json.dumps({"task_id": "HumanEval/0", "prompt": "def f(x):\n"}) + "\n")
    h = et.build_eval_dataset("human_eval", str(he))
    assert h[0]["meta"]["input"] == "def f(x):\n"
    body = et.text_postprocess("```python\ndef f(x):\n    return x + 1\n```\n\nextra", "human_eval")
    assert body.startswith("    ") and "return x + 1" in body and "extra" not in body
    out = tmp_path / "res.jsonl"
    et.save_results(str(out), [{"a": 1}, {"a": 2}])
    assert [json.loads(l)["a"] for l in open(out)] == [1, 2]


def test_interactive_loop_commands():
    """The REPL handles empty input, ``system``, ``clean`` and ``quit`` and keeps the dialogue history."""
    from easyllm_b200.data import build_tokenizer
    from easyllm_b200.engine import PipelineEngine
    from easyllm_b200.infer import generation as gen
    from easyllm_b200.models import llama_custom
    torch.manual_seed(0)
    tok = build_tokenizer({"type": "SimpleTokenizer", "kwargs": {"vocab_size": 512}})
    model = llama_custom(num_layers=1, hidden_size=32, num_attention_heads=2, intermediate_size=64, vocab_size=512,
                         seq_length=128)
    eng = PipelineEngine(model, None, None, {"train_micro_batch_size_per_gpu": 1})
    cfg = {"infer_tokenization": {"type": "sense_tokenization",
                                  "kwargs": {"max_seq_length": 128, "parser_type": "simple_chat",
                                             "parser_kwargs": {"inference_mode": True}}}}
    args = types.SimpleNamespace(out_seq_length=4, temperature=1.0, top_k=0, top_p=0.0, greedy=True, recompute=False)
    script = iter(["", "system", "be brief", "hello", "clean", "hi again", "quit"])
    seen = []

    def fake_input():
        s = next(script)
        seen.append(s)
        return s
    gen.generate_samples_interactive(args, cfg, eng, tok, force_eos_id=None, input_fn=fake_input)
    assert seen[-1] == "quit" and len(seen) == 7


def test_infer_logp_matches_log_softmax(tmp_path):
    """``logp`` mode: per-token label log-probabilities written as jsonl equal a plain log-softmax gather."""
    from easyllm_b200.data import build_tokenizer
    from easyllm_b200.engine import PipelineEngine
    from easyllm_b200.infer import generation as gen
    from easyllm_b200.models import llama_custom
    torch.manual_seed(0)
    tok = build_tokenizer({"type": "SimpleTokenizer", "kwargs": {"vocab_size": 300}})
    model = llama_custom(num_layers=1, hidden_size=32, num_attention_heads=2, intermediate_size=64, vocab_size=300,
                         seq_length=16)
    eng = PipelineEngine(model, None, None, {"train_micro_batch_size_per_gpu": 1})
    g = torch.Generator().manual_seed(3)
    batches = []
    for _ in range(2):
        ids = torch.randint(0, 300, (1, 17), generator=g)
        labels = ids[:, 1:].clone()
        labels[0, :3] = -100                                   # prompt tokens are ignored
        batches.append({"input_ids": ids[:, :-1], "labels": labels})

    def batch_fn(b):
        t = b["input_ids"]
        pos = torch.arange(t.shape[1]).unsqueeze(0)
        return (t, pos, None), (b["labels"], (b["labels"] != -100).long())
    out = tmp_path / "logp.jsonl"
    gen.infer_logp(eng, tok, iter(batches), batch_fn, str(out), 2)
    rows = [json.loads(l) for l in open(out)]
    assert [r["id"] for r in rows] == [0, 1] and len(rows[0]["logp"]) == 16
    with torch.no_grad():
        for r, b in zip(rows, batches):
            pos = torch.arange(16).unsqueeze(0)
            logits = eng.forward_tokens(b["input_ids"], pos).float()
            lp = torch.log_softmax(logits.view(16, -1), -1)
            lab = b["labels"][0]
            want = torch.where(lab >= 0, lp.gather(1, lab.clamp(min=0)[:, None]).squeeze(1), torch.zeros(16))
            assert torch.allclose(torch.tensor(r["logp"]), want, atol=1e-4)
            assert r["logp"][:3] == [0.0, 0.0, 0.0]


def test_hf_inference_interactive_and_question_file(tmp_path):
    """The HF runner's inference loops on a tiny model: the interactive loop keeps / clears history and stops at
    ``quit``; the evaluation loop writes one line per question and keeps the reference answer next to the reply."""
    import json
    import torch
    from easyllm_b200.data import SimpleTokenizer
    from easyllm_b200.infer.hf_inference import hf_inference
    from easyllm_b200.models.hf_models import CausalLM, HFArch
    torch.manual_seed(0)
    tok = SimpleTokenizer(vocab_size=300)
    model = CausalLM(HFArch(family="llama", vocab_size=300, hidden_size=32, intermediate_size=64, num_hidden_layers=2,
                            num_attention_heads=4)).eval()
    cfg_tok = {"type": "sense_tokenization", "kwargs": {"max_seq_length": 256, "parser_type": "simple_chat",
                                                       "parser_kwargs": {"inference_mode": True}}}
    seen = []
    orig = model.generate

    def spy(ids, **kw):
        seen.append(ids.shape[1])
        return orig(ids, **kw)
    model.generate = spy
    script = iter(["first question", "second question", "clean", "third", "quit"])
    hf_inference({"generation_cfg": {"max_new_tokens": 3}}, model, tok, cfg_tok, torch.device("cpu"),
                 input_fn=lambda: next(script))
    # the second prompt carries the first exchange as history, the one after `clean` does not
    assert len(seen) == 3 and seen[1] > seen[0] and seen[2] < seen[1]

    with open(tmp_path / "q.jsonl", "w") as f:
        f.write(json.dumps({"instruction": "what is 1+1", "input": "", "output": "2"}) + "\n")
        f.write(json.dumps({"instruction": "capital of", "input": " France", "output": "Paris"}) + "\n")
    icfg = {"infer_type": "eval", "eval_task": "base", "question_file": str(tmp_path / "q.jsonl"),
            "result_file": str(tmp_path / "out.jsonl"), "generation_cfg": {"max_new_tokens": 2}}
    hf_inference(icfg, model, tok, cfg_tok, torch.device("cpu"))
    rows = [json.loads(l) for l in open(tmp_path / "out.jsonl")]
    assert [r["id"] for r in rows] == [0, 1] and rows[1]["input"] == "capital of France"
    assert [r["gold"] for r in rows] == ["2", "Paris"] and all(isinstance(r["answer"], str) for r in rows)
