"""Command-line surface of the runners.

Parity: llm/utils/general/parser_helper.py:22-132 (training / inference / medusa /
distributed groups).  The ``--deepspeed`` / ``--deepspeed_config`` flags that the
reference obtains from ``deepspeed.add_config_arguments`` are accepted for script
compatibility; the engine here is native, so they only toggle nothing.
"""
from __future__ import annotations

import argparse


def build_parser(extra_args_provider=None):
    p = argparse.ArgumentParser(description="easyllm_b200 arguments", allow_abbrev=False)
    g = p.add_argument_group("training")
    g.add_argument("--config", default=None, help="settings in yaml format")
    g.add_argument("--distribute-checkpointed-activations", action="store_true")
    g.add_argument("--lora-mode", action="store_true")
    g.add_argument("--seed", type=int, default=None)
    g.add_argument("--fp16", action="store_true")
    g.add_argument("--bf16", action="store_true")
    g.add_argument("--opts", type=str, default=None, nargs=argparse.REMAINDER)
    g.add_argument("--port", type=int, default=13333)

    g = p.add_argument_group("inference")
    g.add_argument("--inference", action="store_true")
    g.add_argument("--generate-log-frequency", type=int, default=-1)
    g.add_argument("--generate-mode", type=str, default=None, choices=[None, "interactive", "eval", "logp"])
    g.add_argument("--logp-file", type=str, default="logp.jsonl")
    g.add_argument("--question-file", type=str, default=None)
    g.add_argument("--sample-file", type=str, default="samples.jsonl")
    g.add_argument("--eval_task", type=str, default="base")
    g.add_argument("--force_eos_id", type=int, default=None)
    g.add_argument("--temperature", type=float, default=1.0)
    g.add_argument("--greedy", action="store_true", default=False)
    g.add_argument("--top-p", type=float, default=0.0)
    g.add_argument("--top-k", type=int, default=0)
    g.add_argument("--out-seq-length", type=int, default=1024)
    g.add_argument("--recompute", action="store_true",
                   help="recompute the full prefix for every generated token instead of using the KV cache")
    g.add_argument("--infer-file", type=str, default=None)
    g.add_argument("--predictions-results", type=str, default="predictions_results.json")
    g.add_argument("--with-infer-tokenization", action="store_true")

    g = p.add_argument_group("medusa")
    g.add_argument("--medusa-generate", action="store_true")
    g.add_argument("--medusa-temperature", type=float, default=0.7)
    g.add_argument("--medusa-max-steps", type=int, default=512)
    g.add_argument("--medusa-choices", type=str, default="mc_sim_7b_3_head_top5")
    g.add_argument("--medusa-posterior-threshold", type=float, default=0.09)
    g.add_argument("--medusa-posterior-alpha", type=float, default=0.3)

    g = p.add_argument_group("distributed")
    g.add_argument("--launcher", type=str, default="torch", choices=["slurm", "torch", "mpi"])
    g.add_argument("--tensor-model-parallel-size", type=int, default=None)
    g.add_argument("--pipeline-model-parallel-size", type=int, default=None)
    g.add_argument("--distributed-backend", default="nccl", choices=["nccl", "gloo"])
    g.add_argument("--local_rank", "--local-rank", type=int, default=None)
    g.add_argument("--lazy-mpu-init", type=bool, required=False)

    g = p.add_argument_group("engine (accepted for launch-script compatibility)")
    g.add_argument("--deepspeed", action="store_true")
    g.add_argument("--deepspeed_config", type=str, default=None)
    if extra_args_provider is not None:
        p = extra_args_provider(p)
    return p


def parse_args(argv=None, extra_args_provider=None, ignore_unknown_args=False):
    p = build_parser(extra_args_provider)
    if ignore_unknown_args:
        args, _ = p.parse_known_args(argv)
    else:
        args = p.parse_args(argv)
    return args
