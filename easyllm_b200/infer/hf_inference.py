"""Inference loops of the HF-style runner (llm/utils/general/hf_utils.py:210-383): interactive
chat with history, and sharded dataset evaluation with results gathered on rank 0."""
from __future__ import annotations


import torch
import torch.distributed as dist

from ..utils.log import default_logger as logger


def _tokenization(cfg_tok, tokenizer):
    from ..data.parsers import build_augmentation
    t = build_augmentation([cfg_tok], tokenizer).transforms[0]
    t.parser.inference_mode = True
    return t


def generate_text(model, tokenizer, tokens, device, gen_cfg):
    ids = torch.tensor([tokens], dtype=torch.long, device=device)
    out = model.generate(ids, max_new_tokens=gen_cfg.get("max_new_tokens", 512), do_sample=gen_cfg.get("do_sample", False),
                         temperature=gen_cfg.get("temperature", 1.0), top_k=gen_cfg.get("top_k", 0),
                         top_p=gen_cfg.get("top_p", 0.0), repetition_penalty=gen_cfg.get("repetition_penalty", 1.0),
                         eos_token_id=tokenizer.eos_token_id)
    new = out[0, len(tokens):].tolist()
    if tokenizer.eos_token_id in new:
        new = new[:new.index(tokenizer.eos_token_id)]
    return tokenizer.decode(new, skip_special_tokens=True)


def hf_inference(infer_cfg, model, tokenizer, cfg_tokenization, device, args=None, input_fn=input):
    tok = _tokenization(cfg_tokenization, tokenizer)
    gen_cfg = infer_cfg.get("generation_cfg", {})
    mode = getattr(args, "generate_mode", None) or infer_cfg.get("infer_type", "interactive")
    if mode == "interactive":
        history = []
        while True:
            logger.info("Input your questions (quit to exit) >>> ")
            text = input_fn()
            if text == "quit":
                return
            if text == "clean":
                history = []
                continue
            parser = tok.parser
            meta = parser.build_inference_meta(text, history) if hasattr(parser, "build_inference_meta") else {"text": text}
            tokens, _ = tok(meta)
            reply = generate_text(model, tokenizer, tokens, device, gen_cfg)
            logger.info(f"EasyLLM: {reply}")
            history += [{"role": "user", "content": text}, {"role": "assistant", "content": reply}]
    else:
        from .eval_tasks import build_eval_dataset, evaluate, save_results
        rank = dist.get_rank() if dist.is_initialized() else 0
        world = dist.get_world_size() if dist.is_initialized() else 1
        ds = build_eval_dataset(infer_cfg.get("eval_task", "base"), infer_cfg.get("question_file"), tok)
        results = []
        for i in range(rank, len(ds), world):
            item = ds[i]
            # `answer` becomes the model's reply; the reference answer of the question file is kept as `gold`
            results.append(dict(item["meta"], id=i, gold=item["meta"].get("answer", ""),
                                answer=generate_text(model, tokenizer, item["tokens"], device, gen_cfg)))
        if world > 1:
            from ..parallel.hf_dist import all_gather_object
            results = [r for part in all_gather_object(results) for r in part]
        if rank == 0:
            results.sort(key=lambda r: r["id"])
            save_results(infer_cfg.get("result_file", "results.jsonl"), results)
            evaluate(infer_cfg.get("eval_task", "base"), results)
