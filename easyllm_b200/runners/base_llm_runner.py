"""Megatron-style 3D-parallel runner: ``python -m easyllm_b200.runners.base_llm_runner --config x.yaml``.

Parity: llm/runners/base_llm_runner.py:38-454.  Build order: config components → distributed
env (TP × PP × DP grid, seeds) → ``--opts`` merge → micro-batch calculator → tokenizer → hooks →
model (+LoRA, trainable-parameter selection) → optimizer + LR schedule → engine → checkpoint
load → data.  ``train()`` runs the hook-instrumented loop over ``engine.train_batch``;
``generate()`` serves the interactive / eval / logp modes.

The YAML surface of the reference is kept (``runtime``, ``deepspeed.config``, ``tokenizer``,
``data``, ``trainer``, ``saver``, ``loader``, ``hooks``, ``lora``, ``model``); the ``deepspeed``
block configures the native engine (ZeRO stage, gradient clipping, bf16 / fp16).  Extra
``runtime`` keys: ``fused_tp`` (default true: fused all-gather→GEMM / GEMM→reduce-scatter
kernels when TP > 1 on GPUs), ``nan_policy`` (count | skip | abort), ``watchdog``.
"""
from __future__ import annotations

import time

import torch
import torch.distributed as dist

from ..ckpt.helper import load_checkpoint, save_checkpoint
from ..config import load_yaml, merge_opts_into_cfg, parse_args
from ..data import build_batch_pipe_fn, build_data_iterator, build_tokenizer
from ..engine.pipeline import initialize as engine_initialize
from ..models import build_model
from ..models.lora import log_trainable_params, set_train_params
from ..optim import (build_learning_rate_scheduler, build_num_microbatches_calculator, build_optimizer,
                     get_train_iters)
from ..parallel.grid import get_grid, initialize_distributed
from ..parallel.rng import set_random_seed
from ..utils.log import default_logger as logger
from .hooks import build_hooks

_TRAIN_START_TIME = time.time()


class BaseRunner:
    def __init__(self, args, cfg=None, training=True, base_type="train"):
        self.args, self.config, self.training, self.base_type = args, cfg, training, base_type
        self.build()

    def build(self):
        self.set_param_components()
        self.build_env()
        if getattr(self.args, "opts", None):
            self.config = merge_opts_into_cfg(self.args.opts, self.config)
        self.build_num_microbatches_calculator()
        self.build_tokenizer()
        self.build_hooks()
        self.build_model()
        self.build_trainer()
        self.engine_init()
        self.load_checkpoint()
        self.build_data_engine()

    # ---- configuration ------------------------------------------------------------------------
    def _default_infer_data(self):
        """``data.infer`` of a config written for training only: interactive generation, one prompt per batch,
        the token batch function (what the reference's SFT configs spell out in their ``infer`` block)."""
        data = self.config["data"]
        train = data.get("train") or {}
        data["infer"] = {"seq_length": train.get("seq_length", 2048), "global_batch_size": 1, "micro_batch_size": 1,
                         "infer_type": "interactive",
                         "batch_pipe": {"type": "token_batch_pipe",
                                        "kwargs": {"reset_position_ids": False, "reset_attention_mask": False,
                                                   "eod_mask_loss": False, "loss_on_targets_only": False}}}
        logger.info("config has no data.infer section: using interactive generation with token_batch_pipe")

    def set_param_components(self):
        self.start_iteration = self.consumed_train_samples = self.consumed_train_tokens = 0
        rt = self.config["runtime"]
        if self.base_type == "infer":
            if "infer" not in self.config["data"]:
                self._default_infer_data()
            # inference never touches the training data: build only the infer entry
            self.config["data"]["data_types"] = ["infer"]
        self.deepspeed = rt.get("deepspeed", True)
        cfg_ds = self.config.get("deepspeed") or {"config": {}}
        cfg_ds.setdefault("config", {})
        d = self.config["data"][self.base_type]
        cfg_ds["config"].update(train_micro_batch_size_per_gpu=d["micro_batch_size"],
                                train_batch_size=d.get("global_batch_size", d["micro_batch_size"]))
        self.cfg_engine = cfg_ds
        self.lora_mode = rt.get("lora_mode", False)
        self.cfg_lora = self.config.get("lora")
        if self.lora_mode and self.cfg_lora is None:
            raise ValueError("lora mode must provide the configs of lora!")
        for k in ("fp16", "bf16"):
            if rt.get(k, False) != (cfg_ds["config"].get(k) or {}).get("enabled", False):
                raise ValueError(f"runtime.{k} disagrees with deepspeed.config.{k}.enabled")
        self.micro_batch_size = d["micro_batch_size"]
        self.seq_length = d["seq_length"]

    def build_env(self):
        rt = self.config["runtime"]
        backend = rt.get("distributed_backend", getattr(self.args, "distributed_backend", "nccl"))
        initialize_distributed(tp=rt.get("tensor_model_parallel_size", 1), pp=rt.get("pipeline_model_parallel_size", 1),
                               backend=backend, launcher=getattr(self.args, "launcher", "torch"),
                               port=getattr(self.args, "port", 13333))
        set_random_seed(rt.get("seed", 42), rt.get("dp_random_init", False))
        self.device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() \
            else torch.device("cpu")
        t = torch.tensor([_TRAIN_START_TIME], dtype=torch.float64, device=self.device)
        if dist.is_initialized():
            dist.all_reduce(t, op=dist.ReduceOp.MIN)
        self.start_time = float(t)
        logger.info(f"Initialize env done! Times (seconds): {time.time() - self.start_time:.3f}")

    def build_num_microbatches_calculator(self):
        self.num_microbatches_calculator = None
        if self.training:
            cfg = self.config["data"]["train"].get("batch_calculator") or {
                "type": "constant_num", "kwargs": {"global_batch_size": self.config["data"]["train"]["global_batch_size"],
                                                   "micro_batch_size": self.micro_batch_size}}
            self.num_microbatches_calculator = build_num_microbatches_calculator(cfg)

    def build_tokenizer(self):
        self.tokenizer = build_tokenizer(self.config["tokenizer"], get_grid().tp)

    def build_hooks(self):
        self._hooks = build_hooks(self, self.config.get("hooks", []) if self.training else [],
                                  add_log_if_not_exists=self.training)

    def build_model(self):
        cfg = self.config
        cfg.setdefault("loader", {})
        if not self.training:
            cfg["model"].setdefault("kwargs", {})["sequence_parallel"] = False
            cfg["model"]["kwargs"]["checkpoint_activations"] = False
        model = build_model(self.tokenizer, cfg, self.lora_mode, self.cfg_lora, base_type=self.base_type)
        set_train_params(model, lora_mode=self.lora_mode, cfg_lora=self.cfg_lora, is_train=self.training)
        log_trainable_params(model)
        self.model = model
        rt = cfg["runtime"]
        g = get_grid()
        if g.tp > 1 and rt.get("fused_tp", True) and torch.cuda.is_available() and model.args.bf16 \
                and model.args.sequence_parallel:
            from ..parallel import symm
            symm.install(self.micro_batch_size * self.seq_length, model.args.hidden_size)

    def set_train_iters(self, train_iters):
        self.total_train_iters = get_train_iters(self.num_microbatches_calculator, train_iters,
                                                 self.config["trainer"].get("train_samples"))

    def build_trainer(self):
        self.optimizer = self.lr_scheduler = None
        if not self.training:
            return
        cfg_optim = self.config["trainer"]["optimizer"]
        ds = self.cfg_engine["config"]
        self.optimizer = build_optimizer(cfg_optim, self.model,
                                         zero_stage=(ds.get("zero_optimization") or {}).get("stage", 0),
                                         grad_clip=ds.get("gradient_clipping", 0.0),
                                         fp16=self.config["runtime"].get("fp16", False),
                                         nan_policy=self.config["runtime"].get("nan_policy", "count"),
                                         engine_contract=True)
        cfg_lr = self.config["trainer"]["lr_scheduler"]
        cfg_lr.setdefault("kwargs", {})["max_lr"] = cfg_optim["kwargs"]["lr"]
        if cfg_lr["type"] == "iter_base_annealing":
            cfg_lr["kwargs"]["global_batch_size"] = self.num_microbatches_calculator.global_batch_size
        if cfg_lr["type"] == "hf_cosine":
            cfg_lr["kwargs"].pop("max_lr", None)
        self.lr_scheduler = build_learning_rate_scheduler(cfg_lr, self.optimizer)

    def engine_init(self):
        self.engine, self.optimizer, _, self.lr_scheduler = engine_initialize(
            self.model, self.optimizer, self.lr_scheduler, self.cfg_engine["config"])
        g = get_grid()
        assert self.engine.grid.get_pipe_parallel_rank() == g.pp_rank
        assert self.engine.grid.get_slice_parallel_rank() == g.tp_rank
        assert self.engine.grid.get_data_parallel_rank() == g.dp_rank

    deepspeed_init = engine_init

    def load_checkpoint(self):
        if dist.is_initialized():
            dist.barrier()
        self.start_iteration, self.consumed_train_samples, self.consumed_train_tokens = load_checkpoint(
            self.engine, self.optimizer, self.num_microbatches_calculator, self.config.get("loader"),
            self.lora_mode, self.cfg_lora)
        if hasattr(self.lr_scheduler, "consumed_train_tokens"):
            self.lr_scheduler.consumed_train_tokens = self.consumed_train_tokens
        if hasattr(self.lr_scheduler, "num_steps") and self.consumed_train_samples:
            self.lr_scheduler.num_steps = 0
            self.lr_scheduler.step(self.consumed_train_samples)
        if dist.is_initialized():
            dist.barrier()

    def build_data_engine(self):
        cfg_data = self.config["data"]
        self.data_iterators, self.batch_pipe_func = {}, {}
        dataset_size = 0
        for dt in cfg_data.get("data_types", ["train", "test"]):
            if dt not in ("train", "valid", "test", "infer"):
                raise ValueError("data type only support train, valid, test, and infer")
            self.batch_pipe_func[dt] = build_batch_pipe_fn(cfg_data[dt]["batch_pipe"], self.tokenizer)
            if dt == "infer" and cfg_data[dt].get("infer_type", "interactive") == "interactive":
                continue
            self.data_iterators[dt], dataset_size = build_data_iterator(self.tokenizer, cfg_data,
                                                                        self.consumed_train_samples, dt)
        self.dataset_size = dataset_size
        if self.training:
            epoch = self.config["trainer"].get("epoch", -1)
            if epoch and epoch > 0:
                gbs = self.num_microbatches_calculator.global_batch_size
                iters = int((dataset_size // gbs + 1) * epoch)
            else:
                iters = self.config["trainer"].get("train_iters", 100)
            self.set_train_iters(iters)

    # ---- training -----------------------------------------------------------------------------------
    def save_checkpoint(self, cur_iter, force=False):
        cfg_saver = self.config.get("saver") or {}
        if not cfg_saver.get("save_path"):
            return
        every = cfg_saver.get("save_interval", 0)
        if force or (every and (cur_iter + 1) % every == 0) or (cur_iter + 1 == self.total_train_iters):
            save_checkpoint(cur_iter + 1, self.consumed_train_samples, self.consumed_train_tokens, self.engine,
                            cfg_saver, self.lora_mode, self.cfg_lora)
            logger.info(f"Saving checkpoint at the {cur_iter + 1}_th iter.")

    def forward_step(self, data_iterator):
        loss = self.engine.train_batch(data_iter=data_iterator, dynamic=self.config["runtime"].get("dynamic", False),
                                       sequence_parallel=self.model.sequence_parallel)
        return {"lm_loss": loss}

    def train(self):
        if self.base_type != "train":
            raise ValueError(f"Training type! But the base type is {self.base_type}")
        g = get_grid()
        self._hooks("before_train")
        self.engine.set_batch_fn(self.batch_pipe_func["train"])
        self.model.set_train_status(self.lora_mode)
        output = {}
        for iteration in range(self.start_iteration, self.total_train_iters):
            self._hooks("before_train_iter", iteration)
            self.num_microbatches_calculator.update(self.consumed_train_samples, True)
            gbs = g.dp * self.micro_batch_size * self.num_microbatches_calculator.get()
            self.engine.set_train_batch_size(gbs)
            output = self.forward_step(self.data_iterators["train"])
            self.consumed_train_samples += gbs
            self.consumed_train_tokens += gbs * self.seq_length
            if hasattr(self.lr_scheduler, "consumed_train_tokens"):
                self.lr_scheduler.consumed_train_tokens = self.consumed_train_tokens
            self._hooks("after_train_iter", iteration, output)
            self.save_checkpoint(iteration)
        self._hooks("after_train")
        return output

    # ---- inference ------------------------------------------------------------------------------------
    def generate(self):
        from ..infer.generation import Generator, generate_samples_eval, generate_samples_interactive, infer_logp
        args = self.args
        self.engine.set_batch_fn(self.batch_pipe_func.get("infer"))
        self.model.eval()
        args.out_seq_length = int(self.config["data"]["infer"].get("out_seq_length", args.out_seq_length))
        mode = args.generate_mode or "interactive"
        with torch.no_grad():
            if mode == "interactive":
                generate_samples_interactive(args, self.config, self.engine, self.tokenizer, args.force_eos_id)
            elif mode == "logp":
                infer_logp(self.engine, self.tokenizer, self.data_iterators["infer"], self.batch_pipe_func["infer"],
                           args.logp_file, self.dataset_size // max(1, get_grid().dp))
            elif mode == "eval":
                from ..infer.eval_tasks import run_eval
                run_eval(self, Generator(self.engine, self.tokenizer), generate_samples_eval)
            else:
                raise NotImplementedError(mode)


def main(argv=None):
    args = parse_args(argv)
    if not args.config:
        raise SystemExit("--config is required")
    cfg = load_yaml(args.config)
    rt = cfg.setdefault("runtime", {})
    for key, val in (("seed", args.seed), ("tensor_model_parallel_size", args.tensor_model_parallel_size),
                     ("pipeline_model_parallel_size", args.pipeline_model_parallel_size)):
        if val is not None:
            rt[key] = val
    if args.fp16:
        rt["fp16"] = True
    if args.bf16:
        rt["bf16"] = True
    if args.lora_mode:
        rt["lora_mode"] = True
    rt.setdefault("distributed_backend", args.distributed_backend)
    if args.inference:
        runner = BaseRunner(args, cfg, training=False, base_type="infer")
        runner.generate()
    else:
        runner = BaseRunner(args, cfg, training=True, base_type="train")
        runner.train()
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
