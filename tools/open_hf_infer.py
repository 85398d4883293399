"""Stand-alone inference with an HF-format checkpoint (+ optional LoRA / prompt / prefix adapter), interactive or
over a question file (tools/open_hf_infer.py:27-211 of the reference).

    python tools/open_hf_infer.py --model_path hf_dir [--lora_path adapter] [--family llama] \
        [--tokenizer_type LlamaTokenizer] [--question_file q.jsonl --result_file out.jsonl]
"""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main(argv=None):
    from easyllm_b200.data import build_tokenizer
    from easyllm_b200.infer.hf_inference import generate_text
    from easyllm_b200.models.hf_models import CausalLM
    p = argparse.ArgumentParser()
    p.add_argument("--model_path", required=True)
    p.add_argument("--family", default=None)
    p.add_argument("--lora_path", default=None)
    p.add_argument("--tokenizer_type", default="AutoTokenizer")
    p.add_argument("--tokenizer_path", default=None)
    p.add_argument("--question_file", default=None)
    p.add_argument("--result_file", default="results.jsonl")
    p.add_argument("--max_new_tokens", type=int, default=512)
    p.add_argument("--temperature", type=float, default=0.2)
    p.add_argument("--top_k", type=int, default=40)
    p.add_argument("--top_p", type=float, default=0.9)
    p.add_argument("--do_sample", action="store_true")
    p.add_argument("--dtype", default="bfloat16")
    a = p.parse_args(argv)
    dev = torch.device("cuda" if torch.cuda.is_available() else "cpu")
    tok = build_tokenizer({"type": a.tokenizer_type, "kwargs": {"tokenizer_name_or_path": a.tokenizer_path or a.model_path}})
    model = CausalLM.from_pretrained(a.model_path, family=a.family, torch_dtype=a.dtype if dev.type == "cuda" else "float32")
    soft_dir = None
    if a.lora_path:
        from easyllm_b200.models.lora import merge_lora_into_hf_state
        with open(os.path.join(a.lora_path, "adapter_config.json")) as f:
            c = json.load(f)
        if c.get("peft_type") in ("PROMPT_TUNING", "PREFIX_TUNING"):
            soft_dir, a.lora_path = a.lora_path, None
    if a.lora_path:
        sd = merge_lora_into_hf_state(model.state_dict(), torch.load(os.path.join(a.lora_path, "adapter_model.bin"),
                                                                    map_location="cpu"), c["lora_alpha"] / c["r"])
        model.load_state_dict(sd)
    model = model.to(dev).eval()
    if soft_dir:
        from easyllm_b200.models.hf_models.soft_prompt import load_adapter
        model = load_adapter(model, soft_dir).to(dev).eval()
    gen = dict(max_new_tokens=a.max_new_tokens, temperature=a.temperature, top_k=a.top_k, top_p=a.top_p, do_sample=a.do_sample)
    if a.question_file:
        with open(a.question_file) as f, open(a.result_file, "w") as out:
            for line in f:
                q = json.loads(line)
                text = q.get("instruction", "") + q.get("input", "") or q.get("question", "")
                ans = generate_text(model, tok, tok(text)["input_ids"], dev, gen)
                out.write(json.dumps(dict(q, prediction=ans), ensure_ascii=False) + "\n")
        return
    while True:
        text = input("Input your questions (quit to exit) >>> ")
        if text == "quit":
            break
        print("EasyLLM:", generate_text(model, tok, tok(text)["input_ids"], dev, gen))


if __name__ == "__main__":
    main()
