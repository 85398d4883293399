"""Minimal supervised fine-tuning script over HF-format checkpoints, independent of the YAML runners
(the role of llm/runners/open_hf_runner.py:235-623: an ``HF Trainer`` script for full fine-tuning
or LoRA on llama-family models, reusing this package's datasets and ``batch_align`` collator).

    python -m easyllm_b200.runners.open_hf_runner --model_name_or_path hf_dir --data_path d.jsonl \
        --output_dir out [--use_lora --lora_r 8 --lora_alpha 16] [--num_train_steps 100] [--bf16]
        [--tuning prompt|prefix --num_virtual_tokens 20 [--prompt_init_text "..."]]

Tuning modes: full fine-tuning (default), LoRA (``--use_lora``), prompt tuning and prefix tuning
(``models/hf_models/soft_prompt.py``); the adapters are written in peft's file layout.
Multi-GPU: launch with torchrun (data parallel, ZeRO-1).
"""
from __future__ import annotations

import argparse
import os

import torch
import torch.distributed as dist

from ..data import build_dataset, build_tokenizer
from ..data.collators import BatchAlignCollector
from ..engine.zero_dp import ZeroDPEngine
from ..optim.lr import HFCosineLR
from ..optim.zero import ZeroOptimizer
from ..parallel.grid import initialize_distributed
from ..utils.log import default_logger as logger


def main(argv=None):
    p = argparse.ArgumentParser()
    p.add_argument("--model_name_or_path", required=True)
    p.add_argument("--family", default=None)
    p.add_argument("--tokenizer_type", default="AutoTokenizer")
    p.add_argument("--data_path", required=True)
    p.add_argument("--parser_type", default="simple_chat")
    p.add_argument("--output_dir", required=True)
    p.add_argument("--model_max_length", type=int, default=2048)
    p.add_argument("--per_device_train_batch_size", type=int, default=1)
    p.add_argument("--gradient_accumulation_steps", type=int, default=1)
    p.add_argument("--num_train_steps", type=int, default=100)
    p.add_argument("--learning_rate", type=float, default=2e-5)
    p.add_argument("--weight_decay", type=float, default=0.0)
    p.add_argument("--warmup_steps", type=int, default=10)
    p.add_argument("--bf16", action="store_true")
    p.add_argument("--use_lora", action="store_true")
    p.add_argument("--lora_r", type=int, default=8)
    p.add_argument("--lora_alpha", type=int, default=16)
    p.add_argument("--lora_dropout", type=float, default=0.05)
    p.add_argument("--lora_target", default="q_proj,v_proj")
    p.add_argument("--gradient_checkpointing", action="store_true")
    p.add_argument("--tuning", choices=["none", "prompt", "prefix"], default="none")
    p.add_argument("--num_virtual_tokens", type=int, default=20)
    p.add_argument("--prompt_init_text", default=None)
    a = p.parse_args(argv)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1:
        initialize_distributed(1, 1)
    rank = dist.get_rank() if dist.is_initialized() else 0
    dev = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
    from ..models.hf_models import CausalLM
    from ..models.hf_models.lora import add_lora, save_adapter
    tok = build_tokenizer({"type": a.tokenizer_type, "kwargs": {"tokenizer_name_or_path": a.model_name_or_path}})
    model = CausalLM.from_pretrained(a.model_name_or_path, family=a.family,
                                     torch_dtype=torch.bfloat16 if a.bf16 else torch.float32).to(dev)
    if a.use_lora:
        add_lora(model, {"r": a.lora_r, "lora_alpha": a.lora_alpha, "lora_dropout": a.lora_dropout,
                         "target_modules": a.lora_target.split(",")})
    if a.gradient_checkpointing:
        model.gradient_checkpointing_enable()
    soft = None
    if a.tuning != "none":
        from ..models.hf_models import soft_prompt
        if a.tuning == "prompt":
            init = tok.encode(a.prompt_init_text) if a.prompt_init_text else None
            soft = soft_prompt.PromptTuning(model, a.num_virtual_tokens, init_token_ids=init)
        else:
            soft = soft_prompt.PrefixTuning(model, a.num_virtual_tokens)
        model = soft.to(dev)
    tr = [{"type": "sense_tokenization", "kwargs": {"max_seq_length": a.model_max_length, "parser_type": a.parser_type}}]
    ds = build_dataset({"type": "base_nlp_json", "kwargs": {"json_file": a.data_path, "json_type": "line", "transformer": tr}}, tok)
    coll = BatchAlignCollector(tok, alignment=8, max_seq_length=a.model_max_length, offset_label=False)
    opt = ZeroOptimizer(model.named_parameters(), lr=a.learning_rate, weight_decay=a.weight_decay, stage=1 if world > 1 else 0,
                        grad_clip=1.0)
    sched = HFCosineLR(opt, a.warmup_steps, a.num_train_steps)
    eng = ZeroDPEngine(model, opt, sched, {"gradient_accumulation_steps": a.gradient_accumulation_steps})
    model.train()
    g = torch.Generator().manual_seed(1234)
    step = 0
    while step < a.num_train_steps * a.gradient_accumulation_steps:
        idx = torch.randperm(len(ds), generator=g)[rank::world].tolist()
        for i in range(0, len(idx) - a.per_device_train_batch_size + 1, a.per_device_train_batch_size):
            batch = coll([ds[j] for j in idx[i:i + a.per_device_train_batch_size]])
            out = model(batch["input_ids"].to(dev), batch["attention_mask"].to(dev), labels=batch["labels"].to(dev))
            eng.backward(out["loss"])
            if eng.step() and rank == 0 and eng.global_steps % 10 == 0:
                logger.info(f"step {eng.global_steps}: loss {float(out['loss']):.4f} lr {opt.param_groups[0]['lr']:.2e}")
            step += 1
            if step >= a.num_train_steps * a.gradient_accumulation_steps:
                break
    if rank == 0:
        if soft is not None:
            from ..models.hf_models.soft_prompt import save_adapter as save_soft
            save_soft(soft, a.output_dir)
        elif a.use_lora:
            save_adapter(model, a.output_dir)
        else:
            model.save_pretrained(a.output_dir)


if __name__ == "__main__":
    main()
