"""Medusa runner: train the speculative heads on a frozen base model, then decode with them.

Parity: llm/runners/medusa_runner.py:13-188.  ``python -m easyllm_b200.runners.medusa_runner
--config x.yaml [--inference --medusa-generate]``.  The model config is ``{type: medusa, kwargs:
{base_model: {type, kwargs}, medusa_num_heads, medusa_num_layers, medusa_head_name_or_path}}``;
only ``medusa_head`` parameters train; checkpoints are ``medusa_lm_head.pth``.
"""
from __future__ import annotations

import json
import os
import time

import torch

from ..config import load_yaml, parse_args
from ..models.hf_models.medusa import build_choices
from ..utils.log import default_logger as logger
from .hf_runner import HFRunner


class MedusaRunner(HFRunner):
    def build_model(self):
        super().build_model()
        for n, p in self.model.named_parameters():
            p.requires_grad = n.startswith("medusa_head")
        self.model.base_model.eval()

    def save_checkpoint(self, cfg, global_step):
        if not cfg.get("enabled", True):
            return
        if self.rank == 0:
            out = os.path.join(cfg.get("save_path", "checkpoints"), f"checkpoint-{global_step}")
            os.makedirs(out, exist_ok=True)
            torch.save(self.model.medusa_head.state_dict(), os.path.join(out, "medusa_lm_head.pth"))

    def train(self):
        # the model returns per-head losses; HFRunner.train sums every '*loss*' entry
        orig = self.model.forward

        def fwd(input_ids, attention_mask=None, labels=None, **kw):
            out = orig(input_ids=input_ids, attention_mask=attention_mask, labels=labels, return_dict=True)
            return out._d
        self.model.forward = fwd
        return super().train()

    def infer(self):
        a = self.args
        icfg = self.config.get("infer_cfg", {})
        from ..infer.hf_inference import _tokenization
        tok = _tokenization(self.config["infer_tokenization"], self.tokenizer)
        self.model.eval()
        questions = []
        qf = icfg.get("question_file", getattr(a, "question_file", None))
        if qf:
            with open(qf) as f:
                questions = [json.loads(l) for l in f if l.strip()]
        results = []

        def answer(text):
            parser = tok.parser
            meta = parser.build_inference_meta(text, []) if hasattr(parser, "build_inference_meta") else {"text": text}
            tokens, _ = tok(meta)
            ids = torch.tensor([tokens], device=self.device)
            t0, last = time.time(), None
            for last in self.model.medusa_generate(ids, medusa_generate=a.medusa_generate, temperature=a.medusa_temperature,
                                                   max_steps=a.medusa_max_steps, medusa_choices=a.medusa_choices,
                                                   posterior_threshold=a.medusa_posterior_threshold,
                                                   posterior_alpha=a.medusa_posterior_alpha,
                                                   eos_token_id=self.tokenizer.eos_token_id):
                pass
            new = last["ids"][0, len(tokens):].tolist()
            acc = last["accept_lengths"]
            return (self.tokenizer.decode(new, skip_special_tokens=True),
                    {"count": len(acc), "accept_length": sum(acc) + len(acc), "seconds": time.time() - t0})
        if questions:
            for i, q in enumerate(questions):
                text = q.get("instruction", "") + q.get("input", "")
                out, infos = answer(text)
                results.append({"task_id": i, "input": text, "raw_output": out, "output": out, "answer": q.get("output", ""),
                                "infos": infos})
            steps = sum(r["infos"]["count"] for r in results)
            toks = sum(r["infos"]["accept_length"] for r in results)
            logger.info(f"Forward: {steps}; Accept_length: {toks}; Avg Accept_length: {toks / max(1, steps):.3f}")
            with open(icfg.get("result_file", a.sample_file), "w") as f:
                for r in results:
                    f.write(json.dumps(r, ensure_ascii=False) + "\n")
        else:
            while True:
                text = input("Input your questions (quit to exit) >>> ")
                if text == "quit":
                    break
                out, infos = answer(text)
                logger.info(f"EasyLLM: {out}\n{infos}")
        return results


def main(argv=None):
    args = parse_args(argv)
    cfg = load_yaml(args.config)
    build_choices(args.medusa_choices)          # validate the preset name early
    runner = MedusaRunner(args, cfg, training=not args.inference)
    runner.infer() if args.inference else runner.train()


if __name__ == "__main__":
    main()
