"""Model configuration: the reference's flat ``model.kwargs`` surface → one ``ModelArgs``.

Parity: llm/models/mg_models/llama/default_cfg.py:11-256.  The same flat keys are accepted
(unknown keys are an error), the same five nested override blocks are honoured
(``word_embedings_params``, ``layer_norm_params``, ``transformer_layer_params``,
``lm_head_params``, ``loss_params``) and the same defaults apply: rotary positions, RMSNorm
eps 1e-6, SiLU-GLU, N(0, 0.02) init with N(0, 0.02/sqrt(2L)) for output projections,
``intermediate_size = roundup256(8h/3)`` when unset, ``align_vocab_size_strict`` → ``cut_size``.
Instead of five loosely coupled dicts the result is a single dataclass every layer reads.
"""
from __future__ import annotations

import copy
import math
from dataclasses import dataclass, field
from typing import Any, Dict, Optional

import torch

_SHARED_KEYS = {
    "num_layers": None, "vocab_size": None, "unpad_vocab_size": None, "kv_channels": None,
    "num_attention_heads": None, "num_kv_attention_heads": None, "intermediate_size": None,
    "seq_length": None, "hidden_size": None, "hidden_dropout": 0,
    "position_embedding_type": "rotary", "position_embedding_kwargs": None, "params_dtype": None,
    "pretrain_causal_attention": True, "use_cpu_initialization": False, "parallel_output": True,
    "sync_tp_duplicated_parameters": True, "sequence_parallel": False, "fp16": False, "bf16": False,
    "attn_mask_type": "causal", "fp32_residual_connection": False, "micro_batch_size": 1,
    "use_flash_attn": True,
}
_MODEL_KEYS = {
    "checkpoint_activations": True, "checkpoint_num_layers": 1, "dynamic_checkpoint": None,
    "pp_partition_method": "type:transformer|embedding",
}
_NESTED = ("word_embedings_params", "layer_norm_params", "transformer_layer_params",
           "lm_head_params", "loss_params")
# extensions of this framework (not in the reference surface)
_EXT_KEYS = {"ffn_hidden_size": None, "fused_kernels": True, "fused_lm_head_loss": True}

_DTYPES = {"float32": torch.float32, "fp32": torch.float32, "float": torch.float32,
           "float16": torch.float16, "fp16": torch.float16, "half": torch.float16,
           "bfloat16": torch.bfloat16, "bf16": torch.bfloat16}


@dataclass
class ModelArgs:
    num_layers: int
    hidden_size: int
    num_attention_heads: int
    num_kv_attention_heads: int
    intermediate_size: int
    vocab_size: int
    unpad_vocab_size: Optional[int] = None
    kv_channels: int = 128
    seq_length: Optional[int] = None
    hidden_dropout: float = 0.0
    attention_dropout: float = 0.0
    position_embedding_type: str = "rotary"      # rotary | flash | dynamicntk | alibi | absolute
    rope_base: float = 10000.0
    rope_scale_factor: float = 1.0
    rope_max_position_embeddings: Optional[int] = None
    max_position_embeddings: Optional[int] = None
    params_dtype: torch.dtype = torch.float32
    fp16: bool = False
    bf16: bool = False
    fp32_residual_connection: bool = False
    parallel_output: bool = True
    sync_tp_duplicated_parameters: Any = True     # True | False | "reference"
    sequence_parallel: bool = False
    attn_mask_type: str = "causal"
    use_flash_attn: bool = True
    micro_batch_size: int = 1
    use_cpu_initialization: bool = False
    # norm
    norm_type: str = "rms_norm"
    norm_eps: float = 1e-6
    # block
    glu_activation: Optional[str] = "silu"
    qkv_pack: bool = False
    attention_qkv_bias: bool = False
    attention_o_bias: bool = False
    apply_query_key_layer_scaling: bool = True
    init_sigma: float = 0.02
    output_init_sigma: float = 0.02
    output_init_scaled: bool = True
    embed_init_sigma: float = 0.02
    head_init_sigma: float = 0.02
    # schedule / recompute
    checkpoint_activations: bool = True
    checkpoint_num_layers: int = 1
    dynamic_checkpoint: Optional[Dict] = None
    pp_partition_method: str = "type:transformer|embedding"
    # loss
    loss_type: str = "softmax_cross_entropy"
    loss_kwargs: Dict = field(default_factory=dict)
    # framework switches
    fused_kernels: bool = True
    fused_lm_head_loss: bool = True
    lora: Optional[Dict] = None

    @property
    def head_dim(self):
        return self.kv_channels

    def output_sigma(self):
        if self.output_init_scaled:
            return self.output_init_sigma / math.sqrt(2.0 * self.num_layers)
        return self.output_init_sigma


def resolve_dtype(params_dtype, fp16, bf16):
    if isinstance(params_dtype, torch.dtype):
        dt = params_dtype
    elif params_dtype is None:
        dt = torch.float16 if fp16 else torch.bfloat16 if bf16 else torch.float32
    else:
        dt = _DTYPES[str(params_dtype).replace("torch.", "")]
    if fp16 and dt != torch.float16 or bf16 and dt != torch.bfloat16:
        raise ValueError(f"params_dtype {dt} disagrees with fp16={fp16} bf16={bf16}")
    return dt


def _sigma(init_cfg, default):
    if not init_cfg:
        return default, None
    return (init_cfg.get("kwargs") or {}).get("sigma", default), init_cfg.get("type", "normal")


def update_model_cfg(cfg) -> ModelArgs:
    """Validate + expand the flat kwargs dict of a ``model:`` YAML block into ModelArgs."""
    cfg = copy.deepcopy(cfg)
    nested = {k: (cfg.pop(k, None) or {}) for k in _NESTED}
    lora = cfg.pop("lora", None)
    for k in cfg:
        if k not in _SHARED_KEYS and k not in _MODEL_KEYS and k not in _EXT_KEYS:
            raise KeyError(f"invalid key: {k}")
    sh = dict(_SHARED_KEYS)
    sh.update(_MODEL_KEYS)
    sh.update(_EXT_KEYS)
    sh.update(cfg)
    if sh["ffn_hidden_size"] is not None and sh["intermediate_size"] is None:
        sh["intermediate_size"] = sh["ffn_hidden_size"]
    for need in ("num_layers", "hidden_size", "num_attention_heads"):
        if sh[need] is None:
            raise ValueError(f"model config needs {need}")
    h, nh = sh["hidden_size"], sh["num_attention_heads"]
    if h % nh:
        raise ValueError("hidden_size must be divisible by num_attention_heads")
    if sh["kv_channels"] is None:
        sh["kv_channels"] = h // nh
    elif sh["kv_channels"] != h // nh:
        raise ValueError("kv_channels must equal hidden_size // num_attention_heads")
    if sh["intermediate_size"] is None:
        sh["intermediate_size"] = ((int(2 * (4 * h) / 3) + 255) // 256) * 256
    if sh["num_kv_attention_heads"] is None:
        sh["num_kv_attention_heads"] = nh
    if sh["fp32_residual_connection"] and not (sh["fp16"] or sh["bf16"]):
        raise ValueError("residual connection in fp32 only supported when using fp16 or bf16")
    dtype = resolve_dtype(sh["params_dtype"], sh["fp16"], sh["bf16"])

    emb, ln, tl, head, loss = (nested[k] for k in _NESTED)
    pek = sh["position_embedding_kwargs"] or tl.get("position_embedding_kwargs") or {}
    pet = tl.get("position_embedding_type", sh["position_embedding_type"])
    max_pos = emb.get("max_position_embeddings")
    if pet in ("absolute", "alibi"):
        if max_pos is None:
            raise ValueError(f"position_embedding_type={pet} needs word_embedings_params.max_position_embeddings")
        if sh["seq_length"] is not None and max_pos < sh["seq_length"]:
            raise ValueError("max_position_embeddings < seq_length")
    elif max_pos is not None:
        raise ValueError("max_position_embeddings is only valid with absolute/alibi positions")
    if tl.get("glu_activation", "silu") is not None and tl.get("bias_gelu_fusion", False):
        raise ValueError("if glu-activation is used, please set bias-gelu-fusion to false")
    ln_kwargs = ln.get("kwargs") or {}
    init_sigma, _ = _sigma(tl.get("initializer"), 0.02)
    out_sigma, out_type = _sigma(tl.get("output_initializer"), 0.02)
    emb_sigma, _ = _sigma(emb.get("initializer"), 0.02)
    head_sigma, _ = _sigma(head.get("initializer"), 0.02)
    loss_kwargs = dict(loss.get("kwargs") or {})
    loss_kwargs.setdefault("is_prefix", sh["attn_mask_type"] == "prefix")
    if loss_kwargs.pop("align_vocab_size_strict", False):
        v, uv = sh["vocab_size"], sh["unpad_vocab_size"]
        if v is not None and uv is not None and v != uv:
            loss_kwargs["cut_size"] = v - uv
    if float(tl.get("attention_dropout", 0) or 0) > 0 and tl.get("use_flash_attn", sh["use_flash_attn"]):
        # the fused attention kernels carry no dropout: refuse the combination here, where the config is expanded,
        # instead of training without the dropout the config asks for
        raise ValueError("attention_dropout > 0 needs transformer_layer_params.use_flash_attn: False (the separate "
                         "scores / softmax / value path applies it); the fused attention kernels have no dropout")
    return ModelArgs(
        num_layers=sh["num_layers"], hidden_size=h, num_attention_heads=nh,
        num_kv_attention_heads=sh["num_kv_attention_heads"], intermediate_size=sh["intermediate_size"],
        vocab_size=sh["vocab_size"], unpad_vocab_size=sh["unpad_vocab_size"], kv_channels=sh["kv_channels"],
        seq_length=sh["seq_length"], hidden_dropout=sh["hidden_dropout"],
        attention_dropout=tl.get("attention_dropout", 0),
        position_embedding_type=pet, rope_base=float(pek.get("base", 10000.0)),
        rope_scale_factor=float(pek.get("scale_factor", 1.0)),
        rope_max_position_embeddings=pek.get("max_position_embeddings"),
        max_position_embeddings=max_pos, params_dtype=dtype, fp16=sh["fp16"], bf16=sh["bf16"],
        fp32_residual_connection=sh["fp32_residual_connection"], parallel_output=sh["parallel_output"],
        sync_tp_duplicated_parameters=ln_kwargs.get("sync_tp_duplicated_parameters", sh["sync_tp_duplicated_parameters"]),
        sequence_parallel=sh["sequence_parallel"], attn_mask_type=sh["attn_mask_type"],
        use_flash_attn=tl.get("use_flash_attn", sh["use_flash_attn"]), micro_batch_size=sh["micro_batch_size"],
        use_cpu_initialization=sh["use_cpu_initialization"],
        norm_type=ln.get("type", "rms_norm"), norm_eps=float(ln_kwargs.get("eps", 1e-6)),
        glu_activation=tl.get("glu_activation", "silu"), qkv_pack=tl.get("qkv_pack", False),
        attention_qkv_bias=tl.get("attention_qkv_bias", False), attention_o_bias=tl.get("attention_o_bias", False),
        apply_query_key_layer_scaling=tl.get("apply_query_key_layer_scaling", True),
        init_sigma=init_sigma, output_init_sigma=out_sigma, output_init_scaled=(out_type or "scaled_normal") == "scaled_normal",
        embed_init_sigma=emb_sigma, head_init_sigma=head_sigma,
        checkpoint_activations=sh["checkpoint_activations"], checkpoint_num_layers=sh["checkpoint_num_layers"],
        dynamic_checkpoint=sh["dynamic_checkpoint"], pp_partition_method=sh["pp_partition_method"] or "type:transformer",
        loss_type=loss.get("type", "softmax_cross_entropy"), loss_kwargs=loss_kwargs,
        fused_kernels=sh["fused_kernels"], fused_lm_head_loss=sh["fused_lm_head_loss"], lora=lora,
    )


LLAMA_PRESETS = {
    "llama_7b": dict(num_layers=32, hidden_size=4096, num_attention_heads=32),
    "llama_13b": dict(num_layers=40, hidden_size=5120, num_attention_heads=40),
    "llama_20b": dict(num_layers=60, hidden_size=5120, num_attention_heads=40),
    "llama_65b": dict(num_layers=80, hidden_size=8192, num_attention_heads=64),
    "llama2_7b": dict(num_layers=32, hidden_size=4096, intermediate_size=11008,
                      num_attention_heads=32, num_kv_attention_heads=32),
    "llama2_13b": dict(num_layers=40, hidden_size=5120, intermediate_size=13824,
                       num_attention_heads=40, num_kv_attention_heads=40),
    "llama2_70b": dict(num_layers=80, hidden_size=8192, intermediate_size=28672,
                       num_attention_heads=64, num_kv_attention_heads=8),
    "codellama_7b": dict(num_layers=32, hidden_size=4096, intermediate_size=11008, num_attention_heads=32,
                         num_kv_attention_heads=32, position_embedding_kwargs={"base": 1.0e6}),
    "codellama_13b": dict(num_layers=40, hidden_size=5120, intermediate_size=13824, num_attention_heads=40,
                          num_kv_attention_heads=40, position_embedding_kwargs={"base": 1.0e6}),
    "codellama_34b": dict(num_layers=48, hidden_size=8192, intermediate_size=22016, num_attention_heads=64,
                          num_kv_attention_heads=8, position_embedding_kwargs={"base": 1.0e6}),
}
