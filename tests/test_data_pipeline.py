"""Data layer on CPU: parsers, collators, samplers (resume determinism), index builders
(native C++ vs Python twin), mmap index dataset, batch functions, config loader / opts."""
import json
import os

import numpy as np
import torch

from easyllm_b200.config import load_yaml, merge_opts_into_cfg, clear_include_cache
from easyllm_b200.data import (SimpleTokenizer, build_parser, build_batch_sampler, build_dataset, build_location_idx_py,
                               build_batch_pipe_fn, get_ltor_masks_and_position_ids)
from easyllm_b200.data.collators import BatchAlignCollector, BatchCollector
from easyllm_b200.data.cores import compile as helpers
from easyllm_b200.data.samplers import MegatronPretrainingRandomSampler, MegatronPretrainingSampler

TOK = SimpleTokenizer(vocab_size=32000)


def test_yaml_include_overwrite_and_opts(tmp_path):
    (tmp_path / "base.yaml").write_text("model:\n  kwargs:\n    num_layers: 2\nhooks:\n  - type: a\n    kwargs: {x: 1}\n")
    (tmp_path / "main.yaml").write_text(
        "seed: &s 7\ninc: !include base.yaml//model.kwargs\nall: !include base.yaml\nruntime: {seed: *s}\n"
        "overwrite@:\n  all.hooks.0.kwargs.x: 5\n  all.hooks.1: {type: b}\n  runtime.tp: 2\n")
    clear_include_cache()
    cfg = load_yaml(str(tmp_path / "main.yaml"))
    assert cfg["inc"] == {"num_layers": 2} and cfg["runtime"] == {"seed": 7, "tp": 2}
    assert cfg["all"]["hooks"][0]["kwargs"]["x"] == 5 and cfg["all"]["hooks"][1] == {"type": "b"}
    assert "overwrite@" not in cfg
    out = merge_opts_into_cfg(["runtime.seed", "11", "all.hooks.a-kwargs.x", "2.5", "all.flag", "true",
                               "all.hooks.c-kwargs.y", "z"], cfg)
    assert out["runtime"]["seed"] == 11 and out["all"]["flag"] is True and cfg["runtime"]["seed"] == 7


def test_simple_chat_parser_equivalent_forms():
    p = build_parser("simple_chat", dict(tokenizer=TOK, max_seq_length=512))
    a = p({"instruction": "hi ", "input": "there", "output": "yo"})
    b = p({"messages": [{"role": "user", "content": "hi there"}, {"role": "assistant", "content": "yo"}]})
    c = p([{"role": "user", "content": "hi there"}, {"role": "assistant", "content": "yo"}])
    assert torch.equal(a["input_ids"], b["input_ids"]) and torch.equal(b["input_ids"], c["input_ids"])
    lab = a["labels"]
    n_learn = int((lab != -100).sum())
    assert n_learn == len("yo") + 1 and lab[-1] == TOK.eos_token_id         # answer + EOS supervised only
    multi = p([{"role": "user", "content": "q1"}, {"role": "assistant", "content": "a1"},
               {"role": "user", "content": "q2"}, {"role": "assistant", "content": "a2"},
               {"role": "user", "content": "q3"}, {"role": "assistant", "content": "a3"}])
    # every answer (history and final) is supervised with its EOS; prompts are not
    assert int((multi["labels"] != -100).sum()) == 3 * (2 + 1)
    conv = [{"role": "user", "content": "hi there"}, {"role": "assistant", "content": "yo"}]
    keep = build_parser("simple_chat", dict(tokenizer=TOK, max_seq_length=512, keep_all_keys=True))(conv)
    assert torch.equal(keep["labels"], keep["input_ids"])
    inf = build_parser("simple_chat", dict(tokenizer=TOK, max_seq_length=512, inference_mode=True))
    toks, _ = inf(inf.build_inference_meta("hello"))
    assert toks[-1] != TOK.eos_token_id


def test_truncation_and_drop_meta():
    long_hist = [{"role": "user", "content": "x" * 300}, {"role": "assistant", "content": "y" * 300},
                 {"role": "user", "content": "q"}, {"role": "assistant", "content": "final"}]
    p = build_parser("general_chat", dict(tokenizer=TOK, max_seq_length=256))
    out = p(long_hist)
    assert len(out["input_ids"]) <= 256 and out["labels"][-1] == TOK.eos_token_id
    assert build_parser("general_chat", dict(tokenizer=TOK, max_seq_length=256, drop_meta=True))(long_hist) is None
    base = build_parser("base", dict(tokenizer=TOK, max_seq_length=16))({"text": "z" * 100})
    assert len(base["input_ids"]) == 16 and base["input_ids"][-1] == TOK.eos_token_id


def test_tools_and_dpo_parsers():
    msgs = {"messages": [{"role": "user", "content": "weather?"},
                         {"role": "assistant", "content": "", "tool_calls": [{"function": {"name": "w", "arguments": {}}}]},
                         {"role": "tool", "content": "sunny"}, {"role": "assistant", "content": "sunny!"}],
            "tools": [{"function": {"name": "w", "description": "d"}}]}
    out = build_parser("tools", dict(tokenizer=TOK, max_seq_length=1024))(msgs)
    text = TOK.decode(out["input_ids"].tolist())
    assert "<tools_define>" in text and "<tool_calls_start>" in text and "<tool_response>" in text
    dpo = build_parser("combine_dpo_general_chat", dict(tokenizer=TOK, max_seq_length=256))
    conv = [{"role": "user", "content": "q"}, {"role": "assistant", "content": "good"}]
    conv2 = [{"role": "user", "content": "q"}, {"role": "assistant", "content": "bad!"}]
    sft = dpo({"yw": conv, "yl": conv2, "yw_logp": [1.0], "yl_logp": [1.0]})
    assert sft["scores"].tolist() == [999999, 999999]
    from easyllm_b200.data.parsers import CombinedGeneralChatParser
    n = len(CombinedGeneralChatParser.__call__(dpo, {"convs": conv, "only_last_answer": True})["input_ids"])
    pair = dpo({"yw": conv, "yl": conv2, "yw_logp": [-0.5] * (n - 1), "yl_logp": [-1.0] * (n - 1)})
    assert pair["scores"][0] > pair["scores"][1]


def test_collators_shift_and_pack():
    a = {"input_ids": torch.arange(10), "labels": torch.arange(10)}
    b = {"input_ids": torch.arange(5), "labels": torch.arange(5)}
    out = BatchAlignCollector(TOK, alignment=8, max_seq_length=64)([a, b])
    assert out["input_ids"].shape == (2, 16)
    assert out["input_ids"][0, :9].tolist() == list(range(9)) and out["labels"][0, :9].tolist() == list(range(1, 10))
    assert out["labels"][1, 4].item() == -100 and out["input_ids"][1, 4].item() == len(TOK) - 1
    plain = BatchCollector(TOK, max_seq_length=8)([a, b])
    assert plain["input_ids"].shape == (2, 8) and plain["attention_mask"][1, 5].item() is False
    pre = BatchAlignCollector(TOK, alignment=1, max_seq_length=8, offset_label=False, pretrain=True)
    s1 = {"input_ids": torch.arange(8), "labels": torch.arange(8), "cu_seqlens": torch.tensor([0, 3, 8]),
          "position_ids": torch.tensor([0, 1, 2, 0, 1, 2, 3, 4])}
    packed = pre([s1, s1])
    assert packed["cu_seqlens"].tolist() == [0, 3, 8, 11, 16]


def test_samplers_partition_and_resume():
    seen = []
    for r in range(2):
        s = MegatronPretrainingSampler(20, 0, 2, r, 2)
        seen.append([i for b in s for i in b])
    assert sorted(seen[0] + seen[1]) == list(range(20)) and seen[0][:4] == [0, 1, 4, 5]
    resumed = [i for b in MegatronPretrainingSampler(20, 8, 2, 0, 2) for i in b]
    assert resumed == seen[0][4:]
    full = [b for b in MegatronPretrainingRandomSampler(40, 0, 2, 1, 2)]
    again = [b for b in MegatronPretrainingRandomSampler(40, 16, 2, 1, 2)]
    assert again == full[4:] and all(20 <= i < 40 for b in full for i in b)
    bs = build_batch_sampler({"type": "base", "kwargs": {"sampler": {"type": "dist"}, "total_samples": 10,
                                                          "data_parallel_rank": 0, "data_parallel_size": 2,
                                                          "micro_batch_size": 2}})
    it = iter(bs)
    first = [next(it) for _ in range(4)]
    assert all(len(b) <= 2 for b in first)


def test_location_index_native_matches_python():
    rng = np.random.RandomState(0)
    sizes = rng.randint(1, 50, size=200).astype(np.int32)
    epochs = 3
    doc = np.tile(np.arange(200, dtype=np.int32), epochs)
    rng.shuffle(doc)
    tpe = int(sizes.sum())
    for seq in (4, 17, 64):
        a = helpers.build_location_idx(sizes, doc, seq, epochs, tpe)
        b = build_location_idx_py(sizes, doc, seq, epochs, tpe)
        assert a.dtype == np.int32 and np.array_equal(a, b)
        # every boundary is a valid (document, offset)
        assert (a[:, 1] < sizes[doc[a[:, 0]]]).all()


def test_mmap_index_dataset_roundtrip(tmp_path):
    lines = [json.dumps({"text": "doc %d " % i + "w" * (5 + i % 7)}) for i in range(50)]
    jf = tmp_path / "d.jsonl"
    jf.write_text("\n".join(lines) + "\n")
    tr = [{"type": "sense_tokenization", "kwargs": {"max_seq_length": 4096, "parser_type": "base"}}]
    kw = dict(data_root=str(tmp_path), seed=1, total_samples=30, max_seq_length=32, json_file=str(jf), transformer=tr,
              cache_worker=3, with_cu_lens=True)
    ds_py = build_dataset({"type": "mmap_index_json", "kwargs": dict(kw, cache_location_builder="py")}, TOK)
    assert len(ds_py) >= 30
    item = ds_py[3]
    assert item["input_ids"].shape[0] == 33 and item["cu_seqlens"][-1].item() == 33
    assert len(item["position_ids"]) == 33
    os.remove([str(p) for p in (tmp_path / "train_data_cache").iterdir() if "location_idx" in p.name][0])
    ds_cpp = build_dataset({"type": "mmap_index_json", "kwargs": dict(kw, cache_location_builder="cpp")}, TOK)
    assert all(torch.equal(ds_py[i]["input_ids"], ds_cpp[i]["input_ids"]) for i in range(0, 30, 5))
    js = build_dataset({"type": "base_nlp_json", "kwargs": {"json_file": str(jf), "json_type": "line", "transformer": tr}}, TOK)
    mm = build_dataset({"type": "mmap_json", "kwargs": {"json_file": str(jf), "transformer": tr,
                                                         "cache_dir": str(tmp_path / "c")}}, TOK)
    assert len(js) == len(mm) == 50 and torch.equal(js[7]["input_ids"], mm[7]["input_ids"])


def test_pretrain_bin_dataset(tmp_path):
    shard = np.arange(300, dtype=np.uint16)
    shard[[49, 120]] = TOK.eos_token_id
    np.save(tmp_path / "300_0.npy", shard)
    (tmp_path / "list.txt").write_text(str(tmp_path / "300_0.npy") + "\n")
    tr = [{"type": "sense_tokenization", "kwargs": {"max_seq_length": 100, "parser_type": "pretrain_bin"}}]
    ds = build_dataset({"type": "pretrain_bin", "kwargs": {"txt_files": str(tmp_path / "list.txt"), "bin_size": 300,
                                                           "seq_length": 100, "transformer": tr}}, TOK)
    assert len(ds) == 3
    s0 = ds[0]
    assert s0["cu_seqlens"].tolist() == [0, 50, 100] and s0["position_ids"][50].item() == 0


def test_batch_fn_masks_and_documents():
    eod = len(TOK) - 1
    tok = torch.tensor([[5, 6, eod, 7, 8, 9, eod, 3]])
    mask, loss_mask, pos, cu = get_ltor_masks_and_position_ids(tok, eod, True, True, True)
    assert mask is None and pos.tolist() == [[0, 1, 2, 0, 1, 2, 3, 0]] and cu.tolist() == [0, 3, 7, 8]
    assert loss_mask.tolist() == [[1, 1, 0, 1, 1, 1, 0, 1]]
    fn = build_batch_pipe_fn({"type": "flash_batch_pipe"}, TOK)
    (t, p, m), (lab, lm) = fn({"input_ids": tok, "labels": tok})
    assert torch.equal(m, tok.ne(eod)) and torch.equal(lm, m)


def test_preprocess_reward_mini_rlhf_parsers():
    pre = build_parser("preprocess", dict(tokenizer=TOK, max_seq_length=64))
    out = pre({"inputs": "question: ", "outputs": "answer"})
    n_in = len(TOK.encode("question: "))
    assert out["labels"][:n_in].tolist() == [-100] * n_in and out["labels"][-1] == TOK.eos_token_id
    assert TOK.decode(out["input_ids"].tolist()) == "question: answer"
    keep = build_parser("preprocess", dict(tokenizer=TOK, max_seq_length=64, keep_all_keys=True))({"inputs": "a", "outputs": "b"})
    assert (keep["labels"] != -100).all()

    rw = build_parser("reward", dict(tokenizer=TOK, max_seq_length=32))
    good, bad = rw({"input_text": "prompt ", "choice": "nice", "bad_answer": "awful"})["input_ids"]
    n_q = len(TOK.encode("prompt "))
    assert good[:n_q].tolist() == bad[:n_q].tolist() and good[-1] == bad[-1] == TOK.eos_token_id
    assert TOK.decode(good.tolist()) == "prompt nice" and TOK.decode(bad.tolist()) == "prompt awful"
    rw_inf = build_parser("reward", dict(tokenizer=TOK, max_seq_length=8, inference_mode=True))
    inf = rw_inf({"input_text": "a long prompt that is cut from the left", "choice": "ok"})
    assert len(inf["input_ids"]) == 8 and TOK.decode(inf["input_ids"].tolist()).endswith("ok")
    assert (inf["labels"][-2:] != -100).all() and (inf["labels"][:-2] == -100).all()

    rl = build_parser("mini_rlhf", dict(tokenizer=TOK, max_seq_length=64))
    out = rl({"question": "q? ", "answers": ["first", "second one"], "scores": [0.9, 0.1]})
    assert len(out["input_ids"]) == 2 and torch.allclose(out["scores"], torch.tensor([0.9, 0.1]))
    for ids, lab in zip(out["input_ids"], out["labels"]):
        assert ids[-1] == TOK.eos_token_id and (lab[:len(TOK.encode("q? "))] == -100).all() and lab[-1] == TOK.eos_token_id
    assert build_parser("mini_rlhf", dict(tokenizer=TOK, max_seq_length=64, inference_mode=True))({"question": "q"}) == "q"


def test_intern_tools_and_combined_chat_parsers():
    meta = {"messages": [{"role": "system", "content": "be useful"}, {"role": "user", "content": "plot x"},
                         {"role": "assistant", "content": "running",
                          "tool_calls": [{"function": {"name": "python_interpreter", "arguments": {"code": "print(1)"}}}]},
                         {"role": "tool", "name": "python_interpreter", "content": "1"},
                         {"role": "assistant", "content": "done"}],
            "tools": [{"function": {"name": "search", "description": "web"}},
                      {"function": {"name": "python_interpreter", "description": "py"}}],
            "interpreter": [{"name": "python_interpreter", "description": "runs python"}]}
    p = build_parser("intern_tools", dict(tokenizer=TOK, max_seq_length=2048))
    out = p(meta)
    text = TOK.decode(out["input_ids"].tolist())
    assert text.startswith("<|im_start|>system\nbe useful<|im_end|>\n")
    assert "system name=<|interpreter|>\nruns python" in text and 'system name=<|plugin|>\n[{"name": "search"' in text
    assert "python_interpreter" not in text.split("<|plugin|>")[1].split("<|im_end|>")[0]     # not listed as a plugin
    assert "<|action_start|><|interpreter|>\nprint(1)\n<|action_end|>" in text
    assert "environment name=<|interpreter|>\n1<|im_end|>" in text and text.rstrip().endswith("done<|im_end|>")
    learned = TOK.decode(out["input_ids"][out["labels"] != -100].tolist())
    assert "running" in learned and "done" in learned and "plot x" not in learned and "be useful" not in learned
    toks, labels = build_parser("intern_tools", dict(tokenizer=TOK, max_seq_length=2048, inference_mode=True))(meta["messages"][:2])
    assert TOK.decode(toks).endswith("<|im_start|>assistant\n") and labels == []
    try:
        p({"messages": [], "interpreter": [{"name": "bash", "description": ""}]})
        raise AssertionError("a non-python interpreter must be rejected")
    except ValueError:
        pass

    conv = [{"role": "user", "content": "one"}, {"role": "assistant", "content": "first"},
            {"role": "user", "content": "two"}, {"role": "assistant", "content": "second"}]
    comb = build_parser("combine_general_chat", dict(tokenizer=TOK, max_seq_length=512))
    plain = build_parser("general_chat", dict(tokenizer=TOK, max_seq_length=512))

    def learned_text(o):
        return TOK.decode(o["input_ids"][o["labels"] != -100].tolist())
    assert torch.equal(comb(conv)["labels"], plain(conv)["labels"])                      # no per-record switch
    last = comb({"only_last_answer": True, "convs": conv})
    assert "second" in learned_text(last) and "first" not in learned_text(last)
    everything = comb({"keep_all_keys": True, "convs": conv})
    assert (everything["labels"] != -100).sum() > (plain(conv)["labels"] != -100).sum()
    assert "one" in learned_text(everything)


def test_reward_and_mini_rlhf_collators_and_batch_fns():
    from easyllm_b200.config.registry import BATCH_COLLECTOR_REGISTRY
    pad = len(TOK) - 1
    rw = build_parser("reward", dict(tokenizer=TOK, max_seq_length=32))
    items = [rw({"input_text": "p ", "choice": "good answer", "bad_answer": "bad"}),
             rw({"input_text": "another prompt ", "choice": "y", "bad_answer": "nope nope"})]
    coll = BATCH_COLLECTOR_REGISTRY.build({"type": "reward_batch", "kwargs": {"tokenizer": TOK, "max_seq_length": 32}})
    b = coll(items)
    # chosen sequences first, rejected second, one common width
    assert b["input_ids"].shape[0] == 4 and b["input_ids"].shape == b["labels"].shape
    assert b["input_ids"][0, :len(items[0]["input_ids"][0])].tolist() == items[0]["input_ids"][0].tolist()
    assert b["input_ids"][2, :len(items[0]["input_ids"][1])].tolist() == items[0]["input_ids"][1].tolist()
    assert torch.equal(b["attention_mask"], b["input_ids"].ne(pad)) and (b["labels"][b["input_ids"] == pad] == -100).all()

    rl = build_parser("mini_rlhf", dict(tokenizer=TOK, max_seq_length=64))
    ritems = [rl({"question": "q1 ", "answers": ["a", "bb"], "scores": [1.0, 0.0]}),
              rl({"question": "q2 is longer ", "answers": ["ccc", "d"], "scores": [0.3, 0.7]})]
    rcoll = BATCH_COLLECTOR_REGISTRY.build({"type": "mini_rlhf_batch", "kwargs": {"tokenizer": TOK, "alignment": 8,
                                                                                  "max_seq_length": 64}})
    rb = rcoll(ritems)
    assert rb["input_ids"].shape[0] == 4 and rb["input_ids"].shape[1] % 8 == 0
    assert torch.allclose(rb["scores"], torch.tensor([1.0, 0.0, 0.3, 0.7]))
    fn = build_batch_pipe_fn({"type": "mini_rlhf_json_batch_pipe"}, TOK)
    (tokens, pos, mask), (labels, loss_mask, scores) = fn(rb)
    assert torch.equal(tokens, rb["input_ids"]) and torch.allclose(scores, rb["scores"])
    assert pos[0].tolist() == list(range(tokens.shape[1])) and loss_mask.shape == tokens.shape
    assert (loss_mask[tokens == pad] == 0).all()

    jf = build_batch_pipe_fn({"type": "json_batch_pipe", "kwargs": {"dense_mask": True}}, TOK)
    ids = torch.tensor([[5, 6, 7, pad]])
    (t, p, m), (lab, lm) = jf({"input_ids": ids, "labels": ids})
    assert m.shape == (1, 1, 4, 4) and bool(m[0, 0, 0, 1]) and not bool(m[0, 0, 2, 1])        # True = masked, causal
    assert lm.tolist() == [[1.0, 1.0, 1.0, 0.0]]
    hf = build_batch_pipe_fn({"type": "json_batch_pipe", "kwargs": {"dense_mask": True, "hf_atten_mask": True}}, TOK)
    (_, _, mh), _ = hf({"input_ids": ids, "labels": ids})
    assert bool(mh[0, 0, 3, 3]) and not bool(mh[0, 0, 2, 2])                                  # the padded key is masked

    tf = build_batch_pipe_fn({"type": "token_batch_pipe", "kwargs": {"micro_batch_size": 2}}, TOK)
    flat = torch.arange(10, 18)
    (t, p, _), (lab, lm) = tf(flat)
    t, lab = t.cpu(), lab.cpu()
    assert t.tolist() == [[10, 11, 12, 13], [14, 15, 16, 17]]
    assert lab.tolist() == [[11, 12, 13, TOK.eos_token_id], [15, 16, 17, TOK.eos_token_id]]


def test_dist_samplers_and_infinite_batches():
    from easyllm_b200.data.samplers import DistributedSampler, InfiniteBatchSampler, TestDistributedSampler
    # evaluation sampler: a strided split without padding
    parts = [list(TestDistributedSampler(10, r, 3)) for r in range(3)]
    assert parts == [[0, 3, 6, 9], [1, 4, 7], [2, 5, 8]]
    # training sampler: the ranks see disjoint slices of one seeded permutation, padded to equal length
    full = [list(DistributedSampler(10, r, 4)) for r in range(4)]
    assert all(len(p) == 3 for p in full) and len({i for p in full for i in p}) == 10
    # resume inside an epoch: rank 1 continues where 4 globally consumed samples left it
    s = DistributedSampler(10, 1, 4)
    s.set_consumed_samples(4)
    assert list(s) == full[1][1:]
    # next epoch uses another permutation
    s.set_consumed_samples(12)
    nxt = list(s)
    assert len(nxt) == 3 and s.epoch == 1 and nxt != full[1]
    bs = build_batch_sampler({"type": "base", "kwargs": {"sampler": {"type": "dist"}, "total_samples": 10,
                                                         "data_parallel_rank": 0, "data_parallel_size": 2,
                                                         "micro_batch_size": 2}})
    assert isinstance(bs, InfiniteBatchSampler)
    it = iter(bs)
    got = [next(it) for _ in range(5)]                  # 5 samples per rank and epoch: batches of 2, 2, 1, then epoch 2
    assert [len(b) for b in got] == [2, 2, 1, 2, 2] and bs.consumed_samples == 18
    again = build_batch_sampler({"type": "base", "kwargs": {"sampler": {"type": "dist"}, "total_samples": 10,
                                                            "data_parallel_rank": 0, "data_parallel_size": 2,
                                                            "micro_batch_size": 2}})
    again.set_consumed_samples(4)
    assert next(iter(again)) == got[1]


def test_rampup_batch_size_calculator():
    from easyllm_b200.config.registry import BATCH_CALCULATOR_REGISTRY
    import easyllm_b200.optim  # noqa: F401
    calc = BATCH_CALCULATOR_REGISTRY.build({"type": "rampup_batch_size_num", "kwargs": {
        "start_batch_size": 4, "batch_size_increment": 4, "ramup_samples": 40, "global_batch_size": 16,
        "micro_batch_size": 2}})
    seen = []
    for consumed in (0, 9, 14, 27, 28, 41, 1000):
        calc.update(consumed, False)
        seen.append((calc.get_current_global_batch_size(), calc.get()))
    # three increments over 40 samples: a step every 40/3 samples; micro-batches = global / (micro * dp), dp = 1 here
    assert seen == [(4, 2), (4, 2), (8, 4), (12, 6), (12, 6), (16, 8), (16, 8)]
    from easyllm_b200.optim.microbatches import get_train_iters
    # 4 + 4 + 4 + 4 (consumed 16 -> 8) + 8 + 8 (32 -> 12) + 12 (44 > 40) then 16 per step
    assert get_train_iters(calc, train_samples=44 + 5 * 16) == 7 + 5
