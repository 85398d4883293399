"""Llama-architecture decoder as a pipeline of layer specs.

Parity: llm/models/mg_models/llama/llama.py:22-349.  The spec list keeps the reference's
positions because checkpoint layer files are numbered by them (``layer_{idx:02d}-…``):

    0 cast fn · 1 EmbeddingPipe · 2 layout fn · 3 … L+2 transformer blocks · L+3 layout fn ·
    L+4 final norm · L+5 LM head (untied) · L+6 cast fn

Only the layers of this rank's pipeline stage are instantiated.  Instead of a generic
sequential container the stage runs one fused program: embedding → blocks (residual add
folded into the norm kernels, per-layer selective recompute chosen per micro-batch by the
Dynamic Checkpoint table) → final norm → LM head fused with the vocab-parallel loss.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Optional

import torch
import torch.nn as nn
from torch.utils.checkpoint import checkpoint as torch_checkpoint

from .. import ops
from ..config.registry import LOSS_REGISTRY, MODULE_ZOO_REGISTRY
from ..engine.partition import partition_layers
from ..parallel.grid import get_grid
from .config import LLAMA_PRESETS, ModelArgs, update_model_cfg
from .layers import Embedding, LMHead, ParallelTransformerLayer, build_layer_norm, KVCache
from . import losses as _losses  # noqa: F401  (registers the losses)


@dataclass
class LayerSpec:
    typename: str
    index: int
    layer_number: Optional[int] = None
    param_count: int = 0


@dataclass
class StageIO:
    """What crosses a pipeline-stage boundary (and the first stage's parsed batch)."""
    hidden: Optional[torch.Tensor]          # [T_local, h] residual stream
    position_ids: torch.Tensor              # [T] int32
    cu_seqlens: Optional[torch.Tensor]      # [n+1] int32 or None (one document per sample)
    batch: int
    seq: int
    max_seqlen: int
    max_position: int = 0
    row_start: Optional[torch.Tensor] = None  # [T] int32: first token of each token's document (attention mask)
    tokens: Optional[torch.Tensor] = None     # [T] token ids (first stage only)

    def meta(self):
        if self.row_start is None and self.position_ids.is_cuda:
            from ..ops import cuda as cu
            self.row_start = cu.row_start_of(self.cu_seqlens, self.position_ids.numel(), self.position_ids.device)
        return {"position_ids": self.position_ids, "cu_seqlens": self.cu_seqlens, "max_seqlen": self.max_seqlen,
                "batch": self.batch, "max_position": self.max_position, "row_start": self.row_start}


def _block_params(a: ModelArgs):
    h, d = a.hidden_size, a.kv_channels
    n = h * (a.num_attention_heads + 2 * a.num_kv_attention_heads) * d + a.num_attention_heads * d * h
    n += 3 * h * a.intermediate_size + 2 * h
    return n


class _TorchCheckpointEngine:
    """``save`` / ``load`` with ``torch.save`` semantics (the engine object DeepSpeed exposes on a pipeline module)."""

    def save(self, state_dict, path):
        torch.save(state_dict, path)

    def load(self, path, map_location="cpu"):
        return torch.load(path, map_location=map_location, weights_only=False)


class LlamaModelPipe(nn.Module):
    def __init__(self, args: ModelArgs):
        super().__init__()
        g = get_grid()
        self.args = args
        self.num_layers = L = args.num_layers
        self.parallel_output = args.parallel_output
        self.sequence_parallel = args.sequence_parallel and g.tp > 1
        self.specs = self.build_specs()
        self.parts = partition_layers(self.specs, g.pp, args.pp_partition_method,
                                      [s.param_count for s in self.specs])
        self.stage_id = g.pp_rank
        self.lo, self.hi = self.parts[self.stage_id], self.parts[self.stage_id + 1]
        self.loss_fn = LOSS_REGISTRY.build({"type": args.loss_type, "kwargs": args.loss_kwargs})
        # ---- instantiate this stage's layers, keyed by their spec index ----
        self.layers = nn.ModuleDict()
        for spec in self.specs[self.lo:self.hi]:
            mod = self._build(spec)
            if mod is not None:
                self.layers[str(spec.index)] = mod
        self.block_ids = [s.index for s in self.specs[self.lo:self.hi] if s.typename == "ParallelTransformerLayerPipe"]
        self.has_embedding = self.lo <= 1 < self.hi
        self.has_final_norm = self.lo <= L + 4 < self.hi
        self.has_head = self.lo <= L + 5 < self.hi
        # ---- activation recompute (llama.py:62-73, 97-137) ----
        self.checkpoint_interval = args.checkpoint_num_layers if args.checkpoint_activations else 0
        dc = args.dynamic_checkpoint or {}
        self.size_map = {int(k): int(v) for k, v in (dc.get("size_map") or {}).items()} if dc.get("enabled") else None
        self.num_layers_per_pp = math.ceil(L / g.pp)
        self.start_checkpoint_layer_idx = self.num_layers_per_pp * g.pp_rank
        self.last_recompute_count = 0
        self.kv_caches: Optional[Dict[int, KVCache]] = None

    # -------------------------------------------------------------------------------------
    def build_specs(self) -> List[LayerSpec]:
        a, L = self.args, self.args.num_layers
        emb = (a.vocab_size or 0) * a.hidden_size
        specs = [LayerSpec("to_float16", 0), LayerSpec("EmbeddingPipe", 1, param_count=emb), LayerSpec("transpose", 2)]
        for i in range(L):
            specs.append(LayerSpec("ParallelTransformerLayerPipe", 3 + i, layer_number=i, param_count=_block_params(a)))
        specs += [LayerSpec("undo", L + 3), LayerSpec("RMSNorm", L + 4, param_count=a.hidden_size),
                  LayerSpec("EmbedddingPipeNoTied", L + 5, param_count=emb), LayerSpec("float16_to_fp32", L + 6)]
        return specs

    def _build(self, spec: LayerSpec):
        if spec.typename == "EmbeddingPipe":
            return Embedding(self.args)
        if spec.typename == "ParallelTransformerLayerPipe":
            return ParallelTransformerLayer(self.args, spec.layer_number)
        if spec.typename == "RMSNorm":
            return build_layer_norm(self.args)
        if spec.typename == "EmbedddingPipeNoTied":
            return LMHead(self.args)
        return None

    def layer_index_of(self, module_name: str) -> int:
        return int(module_name.split(".")[1])

    # ---- names the reference's checkpoint helpers reach for on a DeepSpeed PipelineModule -------------------
    # (llm/models/mg_models/llama/utils.py:485-548 walks ``forward_funcs`` and saves through ``checkpoint_engine``)
    checkpoint_parallel_write_pipeline = False            # the first DP rank writes every layer file of its stage

    @property
    def forward_funcs(self):
        """This stage's entries of the layer list in order: the module for parameter-bearing specs, the spec's
        type name for the parameter-free ones (casts / transposes)."""
        return [self.layers[str(s.index)] if str(s.index) in self.layers else s.typename
                for s in self.specs[self.lo:self.hi]]

    def ckpt_layer_path(self, ckpt_dir, local_layer_idx):
        """Layer file of entry ``local_layer_idx`` of this stage for this TP rank."""
        from ..ckpt.layer_files import layer_file
        return layer_file(ckpt_dir, self.lo + local_layer_idx, get_grid().tp_rank)

    @property
    def checkpoint_engine(self):
        return _TorchCheckpointEngine()

    # ---- Dynamic Checkpoint ---------------------------------------------------------------
    def get_checkpoint_range(self, n_tokens: int) -> int:
        """Number of leading layers of this stage to recompute for a micro-batch of ``n_tokens``
        tokens (micro-batch size x sequence length, or the packed length): the value of the first
        ``size_map`` key ≥ n_tokens; −1 (all) when none is."""
        for key in sorted(self.size_map):
            if n_tokens <= key:
                return self.size_map[key]
        return -1

    def recompute_plan(self, seq_len: int) -> List[bool]:
        """Per local block: recompute its activations in backward?"""
        n = len(self.block_ids)
        if not self.training or self.checkpoint_interval == 0 and self.size_map is None:
            return [False] * n
        if self.size_map is not None:
            k = self.get_checkpoint_range(seq_len)
            if k < 0:
                return [True] * n
            lim = self.start_checkpoint_layer_idx + k
            return [(bid - 3) < lim for bid in self.block_ids]
        return [True] * n

    # ---- batch parsing ---------------------------------------------------------------------
    def parse_batch(self, inputs, device=None) -> StageIO:
        """First-stage input ``(tokens [b,s], position_ids [b,s], attention_mask[, cu_seqlens])`` → StageIO on
        ``device`` (default: where the tokens are).  Batches from a loader arrive on the host: every scalar the
        kernels need (longest document, highest position, the id range check) is read there, before the copy to
        the GPU, so a training micro-batch costs no device→host synchronisation.  Device-resident inputs with
        ``cu_seqlens`` still work but read those scalars back."""
        if torch.is_tensor(inputs):
            inputs = (inputs,)
        tokens = inputs[0]
        b, s = tokens.shape
        src = tokens.device
        dev = torch.device(device) if device is not None else src
        host = src.type == "cpu"
        if host and self.has_embedding:
            self.layers["1"].word_embeddings.check_ids(tokens)
        max_position = s
        if len(inputs) > 1 and inputs[1] is not None:
            pos = inputs[1].reshape(-1).to(torch.int32)
            if host or inputs[1].device.type == "cpu":
                max_position = max(s, int(pos.max()) + 1 if pos.numel() else 1)
            else:
                max_position = 0                              # resolved below / by the first consumer
        else:
            pos = torch.arange(s, dtype=torch.int32, device=src).repeat(b)
        cu = inputs[3] if len(inputs) > 3 else None
        max_seqlen = s
        if cu is not None:
            cu = cu.reshape(-1).to(torch.int32)
            # collators emit per-sample boundaries offset by sample index; drop repeats / padding
            cu = torch.unique_consecutive(cu)
            if int(cu[-1]) < b * s:
                cu = torch.cat((cu, cu.new_tensor([b * s])))
            max_seqlen = int((cu[1:] - cu[:-1]).max())
        elif b > 1:
            cu = torch.arange(0, (b + 1) * s, s, dtype=torch.int32, device=src)
        if max_position == 0:
            max_position = max(s, int(pos.max()) + 1 if pos.numel() else 1)
        row_start = None
        if dev.type == "cuda":
            from ..ops import cuda as cu_ops
            if cu_ops.available():
                row_start = cu_ops.row_start_of(cu, b * s, dev)

        def mv(t):
            return t if t is None or t.device == dev else t.to(dev, non_blocking=True)
        io = StageIO(None, mv(pos), mv(cu), b, s, max_seqlen, max_position=max_position, row_start=row_start)
        io.tokens = mv(tokens.reshape(-1))
        return io

    # ---- forward of this stage ---------------------------------------------------------------
    def _run_block(self, layer, delta, residual, meta, recompute, kv_cache):
        if recompute and kv_cache is None and torch.is_grad_enabled():
            def fn(d, r):
                return layer(d, r, meta)
            return torch_checkpoint(fn, delta, residual, use_reentrant=False)
        return layer(delta, residual, meta, kv_cache)

    def forward_stage(self, io: StageIO, labels=None, return_logits=False):
        """Runs this stage.  Returns a StageIO (intermediate stage), a scalar loss (last stage
        with ``labels``) or logits ``[b, s, V(/tp)]`` (last stage, ``return_logits``)."""
        g = get_grid()
        a = self.args
        if self.has_embedding:
            x = self.layers["1"](io.tokens, io.position_ids.long())
            if a.fp32_residual_connection:
                x = x.float()
            delta, residual = x, None
        else:
            delta, residual = io.hidden, None
        meta = io.meta()
        plan = self.recompute_plan(io.batch * io.seq)      # Dynamic Checkpoint: keyed on the micro-batch's token count
        self.last_recompute_count = sum(plan)
        for bid, rc in zip(self.block_ids, plan):
            cache = self.kv_caches.get(bid) if self.kv_caches is not None else None
            delta, residual = self._run_block(self.layers[str(bid)], delta, residual, meta, rc, cache)
        if not self.has_final_norm:
            io.hidden = delta if residual is None else delta + residual
            return io
        norm = self.layers[str(self.num_layers + 4)]
        if residual is None:
            x = norm(delta)
        else:
            x, _ = norm(delta, residual)
        head = self.layers[str(self.num_layers + 5)]
        if labels is not None and not return_logits:
            return self.compute_loss(head, x, io, labels)
        logits = head(x)
        return logits.float().view(io.batch, io.seq, -1)

    def compute_loss(self, head, x, io, labels):
        lab = labels[0]
        fused = (self.args.fused_lm_head_loss and type(self.loss_fn).__name__ == "CrossEntropy"
                 and not getattr(head, "lora_head", False))
        if fused:
            # under sequence parallelism the gather of the hidden rows is part of the fused op
            sp = bool(self.args.sequence_parallel) and get_grid().tp > 1
            xin = x if sp else head.gathered_input(x)
            safe = lab.reshape(-1).masked_fill(lab.reshape(-1) == -100, 0)
            tok = ops.lm_head_cross_entropy(xin, head.word_embeddings.weight, safe, self.loss_fn.cut_size,
                                            gather_sp=sp)
            return self.loss_fn.from_token_losses(tok, lab, labels[1])
        logits = head(x).float().view(io.batch, io.seq, -1)
        return self.loss_fn(logits, labels)

    def forward(self, inputs, labels=None, return_logits=False):
        """Single-stage convenience: batch tuple in, loss / logits out."""
        io = self.parse_batch(inputs) if not isinstance(inputs, StageIO) else inputs
        return self.forward_stage(io, labels, return_logits)

    # ---- inference helpers -------------------------------------------------------------------
    def allocate_kv_cache(self, batch, max_len):
        a, g = self.args, get_grid()
        dev = next(self.parameters()).device
        self.kv_caches = {bid: KVCache(batch, max_len, a.num_kv_attention_heads // g.tp, a.kv_channels,
                                       a.params_dtype, dev) for bid in self.block_ids}

    def free_kv_cache(self):
        self.kv_caches = None

    def set_train_status(self, lora_mode=False):
        self.train()
        if lora_mode:
            for n, m in self.named_modules():
                if not any(True for _ in m.children()) and not any("lora_" in pn for pn, _ in m.named_parameters()):
                    m.eval()


def llama_custom(**cfg_model):
    args = cfg_model.pop("model_args", None) or update_model_cfg(cfg_model)
    return LlamaModelPipe(args)


def _preset(name):
    def build(**cfg_model):
        preset = LLAMA_PRESETS[name]
        for k, v in preset.items():
            if k in cfg_model and cfg_model[k] != v:
                raise ValueError(f"{name}: {k}={cfg_model[k]} conflicts with the preset value {v}")
        merged = dict(cfg_model)
        merged.update(preset)
        return llama_custom(**merged)
    build.__name__ = name
    return build


MODULE_ZOO_REGISTRY.register("llama_custom", llama_custom)
for _n in LLAMA_PRESETS:
    MODULE_ZOO_REGISTRY.register(_n, _preset(_n))


def get_layer_info(cfg_model):
    kind, kw = cfg_model["type"], cfg_model.get("kwargs") or {}
    n = LLAMA_PRESETS[kind]["num_layers"] if kind in LLAMA_PRESETS else kw["num_layers"]
    return n, kw.get("checkpoint_num_layers", 1)


def build_model(tokenizer, cfg, lora_mode=False, cfg_lora=None, base_type="train"):
    """llm/models/mg_models/__init__.py:29-53: inject vocab / dtype / batch geometry from the
    tokenizer and runtime config, check qkv_pack ↔ loader.pretrain_type, build, add LoRA."""
    cfg_model = cfg["model"]
    kw = cfg_model.setdefault("kwargs", {})
    padded = getattr(tokenizer, "padded_vocab_size", None)
    vocab = padded if padded is not None and padded != len(tokenizer) else len(tokenizer)
    kw.update({"fp16": cfg["runtime"].get("fp16", False), "bf16": cfg["runtime"].get("bf16", False),
               "unpad_vocab_size": getattr(tokenizer, "vocab_size", vocab), "vocab_size": vocab,
               "micro_batch_size": cfg["data"][base_type]["micro_batch_size"],
               "seq_length": cfg["data"][base_type]["seq_length"]})
    packed = (kw.get("transformer_layer_params") or {}).get("qkv_pack", False)
    pretrain_type = (cfg.get("loader") or {}).get("pretrain_type", "llama")
    if packed and "pack" not in pretrain_type:
        raise ValueError("qkv_pack must load the model in pack type (llama_pack / internlm2_pack)")
    if not packed and "pack" in pretrain_type:
        raise ValueError("the loader uses a pack type but transformer_layer_params.qkv_pack is not set")
    model = MODULE_ZOO_REGISTRY.build(cfg_model)
    if lora_mode and cfg_lora is not None:
        from .lora import convert_layer_to_lora
        model = convert_layer_to_lora(model, cfg_lora)
    return model
