"""Tensor/sequence-parallel building blocks of the Llama-architecture decoder.

Activations are token-major 2-D ``[T, hidden]`` (``T = batch·seq``; packed documents are
described by ``cu_seqlens``), sequence parallelism shards ``T`` over the TP group.  The
projections of a block are held fused — one ``q|k|v`` weight and one ``gate|up`` weight per
rank — so each is one GEMM (and one sequence-parallel all-gather) instead of three / two;
``state_dict`` still exposes the reference's names (``self_attn.{q,k,v}_proj.weight`` or
``self_attn.wqkv.weight``, ``mlp.{gate,up}_proj.weight``) so checkpoints stay compatible.

Parity map (reference file → class here):
  base_modules/layers/column_parallel_linear.py:162-266   → ColumnParallelLinear
  base_modules/layers/row_parallel_linear.py:11-132       → RowParallelLinear
  base_modules/layers/vocab_parallel_emb.py:34-137        → VocabParallelEmbedding
  base_modules/layers/fused_layer_norm.py:20-155          → RMSNorm / LayerNorm / build_layer_norm
  llama/transformer.py:146-225, 228-597, 625-867          → ParallelMLP / ParallelAttention / ParallelTransformerLayer
  llama/word_embedings.py:11-177, llama/lm_head.py:49-104 → Embedding / LMHead
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from ..ops import reference as ref
from ..parallel import mappings as mp
from ..parallel.grid import get_grid
from ..parallel.rng import get_rng_tracker
from ..parallel.tp_linear import column_parallel_linear, row_parallel_linear
from .config import ModelArgs


def _device():
    return torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")


def _tag(p, is_parallel, dim, stride=1):
    """TP attributes consumed by the checkpoint code and the grad-norm/clip logic
    (llm/utils/model/initializer.py:30-66)."""
    p.tensor_model_parallel = is_parallel
    p.partition_dim = dim
    p.partition_stride = stride
    return p


def _init_normal_(w, sigma, sharded):
    if sharded:
        with get_rng_tracker().fork():
            nn.init.normal_(w, mean=0.0, std=sigma)
    else:
        nn.init.normal_(w, mean=0.0, std=sigma)


class ColumnParallelLinear(nn.Module):
    """``Y = X·Aᵀ`` with A split along its rows (output features).  ``segments`` lists named
    global sub-matrices that are each split over TP and stored concatenated on this rank."""

    def __init__(self, in_features, out_features=None, bias=False, gather_output=False, sequence_parallel=False,
                 sigma=0.02, dtype=torch.float32, segments=None, skip_init=False):
        super().__init__()
        tp = get_grid().tp
        if segments is None:
            segments = [("weight", out_features)]
        self.segments = [(n, s) for n, s in segments]
        for n, s in self.segments:
            if s % tp:
                raise ValueError(f"{n}: {s} output features are not divisible by tensor-parallel size {tp}")
        self.local_sizes = [s // tp for _, s in self.segments]
        self.in_features = in_features
        self.out_features = sum(s for _, s in self.segments)
        self.out_local = sum(self.local_sizes)
        self.gather_output = gather_output
        self.sequence_parallel = sequence_parallel and tp > 1
        self.weight = _tag(nn.Parameter(torch.empty(self.out_local, in_features, dtype=dtype, device=_device())), True, 0)
        self.bias = _tag(nn.Parameter(torch.zeros(self.out_local, dtype=dtype, device=_device())), True, 0) if bias else None
        if not skip_init:
            _init_normal_(self.weight.data, sigma, sharded=tp > 1)

    def forward(self, x):
        y = column_parallel_linear(x, self.weight, self.bias, self.sequence_parallel)
        if self.gather_output:
            y = mp.gather_from_tensor_model_parallel_region(y)
        return y


class RowParallelLinear(nn.Module):
    """``Y = X·Aᵀ`` with A split along its columns (input features); the partial products are
    reduce-scattered (SP) or all-reduced over TP.  Bias is replicated and added after."""

    def __init__(self, in_features, out_features, bias=False, input_is_parallel=True, sequence_parallel=False,
                 sigma=0.02, dtype=torch.float32, skip_init=False):
        super().__init__()
        tp = get_grid().tp
        if in_features % tp:
            raise ValueError(f"{in_features} input features are not divisible by tensor-parallel size {tp}")
        self.in_features, self.out_features = in_features, out_features
        self.in_local = in_features // tp
        self.input_is_parallel = input_is_parallel
        self.sequence_parallel = sequence_parallel and tp > 1
        self.weight = _tag(nn.Parameter(torch.empty(out_features, self.in_local, dtype=dtype, device=_device())), True, 1)
        self.bias = _tag(nn.Parameter(torch.zeros(out_features, dtype=dtype, device=_device())), False, -1) if bias else None
        if self.bias is not None:
            self.bias.sequence_parallel = self.sequence_parallel
        if not skip_init:
            _init_normal_(self.weight.data, sigma, sharded=tp > 1)

    def forward(self, x):
        if not self.input_is_parallel:
            x = mp.scatter_to_tensor_model_parallel_region(x)
        return row_parallel_linear(x, self.weight, self.bias, self.sequence_parallel)


class VocabParallelEmbedding(nn.Module):
    """Embedding table split along the vocabulary: ids outside this rank's range contribute
    zeros, the partial lookups are summed over TP."""

    def __init__(self, num_embeddings, embedding_dim, sigma=0.02, dtype=torch.float32, skip_init=False):
        super().__init__()
        g = get_grid()
        if num_embeddings % g.tp:
            raise ValueError(f"vocab size {num_embeddings} is not divisible by tensor-parallel size {g.tp}")
        self.num_embeddings, self.embedding_dim = num_embeddings, embedding_dim
        self.per_rank = num_embeddings // g.tp
        self.vocab_start = g.tp_rank * self.per_rank
        self.vocab_end = self.vocab_start + self.per_rank
        self.weight = _tag(nn.Parameter(torch.empty(self.per_rank, embedding_dim, dtype=dtype, device=_device())), True, 0)
        if not skip_init:
            _init_normal_(self.weight.data, sigma, sharded=g.tp > 1)

    def check_ids(self, ids):
        """Token ids must lie inside the table.  CPU tensors are checked here; on the GPU the lookup kernel checks
        every id itself and reports through the device error word (no ``max()`` read-back per micro-batch)."""
        if not ids.is_cuda and ids.numel():
            hi, lo = int(ids.max()), int(ids.min())
            if hi >= self.num_embeddings or lo < 0:
                raise ValueError(f"An input token id {hi if hi >= self.num_embeddings else lo} is out of bounds of "
                                 f"the embedding table (vocab size {self.num_embeddings})")

    def lookup(self, ids):
        """Local partial lookup (no reduction): rows for foreign ids are zero."""
        if self.weight.is_cuda and self.weight.dtype == torch.bfloat16:
            return ops.embedding(ids, self.weight, self.vocab_start, self.num_embeddings)
        if get_grid().tp == 1:
            return F.embedding(ids, self.weight)
        mask = (ids < self.vocab_start) | (ids >= self.vocab_end)
        local = (ids - self.vocab_start).masked_fill(mask, 0)
        out = F.embedding(local, self.weight)
        return out.masked_fill(mask.unsqueeze(-1), 0.0)

    def forward(self, ids):
        self.check_ids(ids)
        if ids.is_cuda and not (self.weight.dtype == torch.bfloat16) and ids.numel() and \
                int(ids.max()) >= self.num_embeddings:       # fp32 / fp16 tables on a GPU take the PyTorch lookup
            raise ValueError(f"An input token id {int(ids.max())} is out of bounds of the embedding table "
                             f"(vocab size {self.num_embeddings})")
        return mp.reduce_from_tensor_model_parallel_region(self.lookup(ids))


class RMSNorm(nn.Module):
    """RMSNorm with fp32 statistics; the weight is replicated over TP.  Under sequence
    parallelism each rank sees a slice of the tokens, so the weight gradient is summed over
    the TP group once per step by the engine (``sequence_parallel`` attribute on the
    parameter) — instead of averaging the weights every forward as the reference does
    (fused_layer_norm.py:51-54); ``sync_mode='reference'`` restores that behaviour."""

    def __init__(self, normalized_shape, eps=1e-6, sequence_parallel=False, sync_mode=True, dtype=torch.float32,
                 hf_mode=False, **_ignored):
        super().__init__()
        self.eps = eps
        self.weight = _tag(nn.Parameter(torch.ones(normalized_shape, dtype=dtype, device=_device())), False, -1)
        self.weight.sequence_parallel = bool(sequence_parallel) and get_grid().tp > 1
        self.sync_mode = sync_mode

    def _maybe_sync(self):
        if self.sync_mode == "reference" and get_grid().tp > 1:
            import torch.distributed as dist
            with torch.no_grad():
                dist.all_reduce(self.weight.data, group=get_grid().tp_group)
                self.weight.data.div_(get_grid().tp)

    def forward(self, x, residual=None):
        self._maybe_sync()
        if residual is None:
            return ops.rmsnorm(x, self.weight, self.eps)
        return ops.add_rmsnorm(x, residual, self.weight, self.eps)


class LayerNorm(nn.Module):
    """Affine LayerNorm with fp32 statistics and fp32 parameter gradients on the sm_100a kernel
    (``ops/csrc/layernorm.cu``; the reference's MixedFusedLayerNorm, fused_layer_norm.py:74-140; unused by the
    Llama presets), optionally fused with the residual add in front of it."""

    def __init__(self, normalized_shape, eps=1e-5, sequence_parallel=False, dtype=torch.float32, **_ignored):
        super().__init__()
        self.eps = eps
        self.weight = _tag(nn.Parameter(torch.ones(normalized_shape, dtype=dtype, device=_device())), False, -1)
        self.bias = _tag(nn.Parameter(torch.zeros(normalized_shape, dtype=dtype, device=_device())), False, -1)
        sp = bool(sequence_parallel) and get_grid().tp > 1
        self.weight.sequence_parallel = sp
        self.bias.sequence_parallel = sp

    def forward(self, x, residual=None):
        return ops.layernorm(x, self.weight, self.bias, self.eps, residual)


def build_layer_norm(args: ModelArgs):
    if args.norm_type in ("rms_norm", "rmsnorm"):
        return RMSNorm(args.hidden_size, eps=args.norm_eps, sequence_parallel=args.sequence_parallel,
                       sync_mode=args.sync_tp_duplicated_parameters, dtype=args.params_dtype)
    if args.norm_type in ("layer_norm", "layernorm", "fused_layer_norm"):
        return LayerNorm(args.hidden_size, eps=args.norm_eps, sequence_parallel=args.sequence_parallel,
                         dtype=args.params_dtype)
    raise ValueError(f"unknown norm type {args.norm_type}")


class RotaryTables:
    """fp32 cos/sin tables ``[pos, D/2]`` grown on demand; linear scaling and dynamic-NTK
    variants of llama/positional_embeddings.py:5-89."""

    def __init__(self, head_dim, base=10000.0, scale_factor=1.0, ntk_max_pos=None):
        self.head_dim, self.base, self.scale, self.ntk_max_pos = head_dim, base, scale_factor, ntk_max_pos
        self.cos = self.sin = None
        self.cached = 0

    def get(self, need, device):
        if self.cos is None or need > self.cached or self.cos.device != device:
            n = max(need, 2048)
            n = 1 << (n - 1).bit_length()
            ntk = self.ntk_max_pos
            if ntk is not None and need <= ntk:
                n = min(n, ntk) if n >= need else n
            self.cos, self.sin = ref.rope_tables(self.head_dim, n, self.base, self.scale, device, ntk)
            self.cached = n
        return self.cos, self.sin


def alibi_slopes(n_heads):
    def pow2(n):
        start = 2 ** (-2 ** -(math.log2(n) - 3))
        return [start * start ** i for i in range(n)]
    if math.log2(n_heads).is_integer():
        return pow2(n_heads)
    c = 2 ** math.floor(math.log2(n_heads))
    return pow2(c) + pow2(2 * c)[0::2][:n_heads - c]


class KVCache:
    """Per-layer key/value cache ``[B, S_max, Hk, D]`` for incremental decoding."""

    def __init__(self, batch, max_len, n_kv, head_dim, dtype, device):
        self.k = torch.zeros(batch, max_len, n_kv, head_dim, dtype=dtype, device=device)
        self.v = torch.zeros_like(self.k)
        self.len = 0


class ParallelAttention(nn.Module):
    def __init__(self, args: ModelArgs, layer_number):
        super().__init__()
        g = get_grid()
        a = args
        self.args = a
        self.layer_number = layer_number
        self.D = a.kv_channels
        if a.num_attention_heads % g.tp or a.num_kv_attention_heads % g.tp:
            raise ValueError("attention heads must be divisible by the tensor-parallel size")
        self.hq = a.num_attention_heads // g.tp
        self.hk = a.num_kv_attention_heads // g.tp
        nq, nk = a.num_attention_heads * self.D, a.num_kv_attention_heads * self.D
        self.qkv = ColumnParallelLinear(a.hidden_size, bias=a.attention_qkv_bias, sequence_parallel=a.sequence_parallel,
                                        sigma=a.init_sigma, dtype=a.params_dtype,
                                        segments=[("q_proj", nq), ("k_proj", nk), ("v_proj", nk)])
        self.o_proj = RowParallelLinear(nq, a.hidden_size, bias=a.attention_o_bias, sequence_parallel=a.sequence_parallel,
                                        sigma=a.output_sigma(), dtype=a.params_dtype)
        self.pos_type = a.position_embedding_type
        self.rotary = None
        if self.pos_type in ("rotary", "flash", "dynamicntk"):
            self.rotary = RotaryTables(self.D, a.rope_base, a.rope_scale_factor,
                                       a.rope_max_position_embeddings if self.pos_type == "dynamicntk" else None)
        self.alibi = None
        if self.pos_type == "alibi":
            sl = alibi_slopes(a.num_attention_heads)[g.tp_rank * self.hq:(g.tp_rank + 1) * self.hq]
            self.alibi = torch.tensor(sl, dtype=torch.float32)
        self._register_state_dict_hook(_split_fused_hook("qkv", "wqkv" if a.qkv_pack else None))
        self.register_load_state_dict_pre_hook(_merge_fused_hook(self.qkv, "qkv", "wqkv" if a.qkv_pack else None))

    def forward(self, x, meta, kv_cache: Optional[KVCache] = None):
        """x: ``[T(/tp), h]``; meta: dict(position_ids [T], cu_seqlens, max_seqlen, batch)."""
        qkv = self.qkv(x)                                    # [T, (hq+2hk)·D]
        T = qkv.shape[0]
        pos = meta["position_ids"]
        rope = None
        if self.rotary is not None:
            need = int(meta.get("max_position", 0)) or (int(pos.max()) + 1 if pos.numel() else 1)
            cos, sin = self.rotary.get(need, qkv.device)
            rope = (cos, sin, pos)
        nq, nk = self.hq * self.D, self.hk * self.D
        if kv_cache is None and self.args.use_flash_attn:
            slopes = self.alibi.to(qkv.device) if self.alibi is not None else None
            o = ops.flash_attention_packed(qkv, self.hq, self.hk, self.D, meta.get("cu_seqlens"),
                                           meta.get("max_seqlen"), alibi_slopes=slopes, rope=rope,
                                           row_start=meta.get("row_start"))
            return self.o_proj(o)
        if rope is not None:
            qkv = ops.rope_packed(qkv, cos, sin, pos, self.hq, self.hk, self.D)
        q = qkv[:, :nq].view(T, self.hq, self.D)
        k = qkv[:, nq:nq + nk].view(T, self.hk, self.D)
        v = qkv[:, nq + nk:].view(T, self.hk, self.D)
        if kv_cache is not None:
            B = meta["batch"]
            S = T // B
            p0 = kv_cache.len
            kv_cache.k[:, p0:p0 + S] = k.reshape(B, S, self.hk, self.D)
            kv_cache.v[:, p0:p0 + S] = v.reshape(B, S, self.hk, self.D)
            kv_cache.len = p0 + S
            o = ref.attention_kvcache(q.reshape(B, S, self.hq, self.D), kv_cache.k[:, :p0 + S],
                                      kv_cache.v[:, :p0 + S], p0).reshape(T, nq)
        else:
            slopes = self.alibi.to(q.device) if self.alibi is not None else None
            if not self.args.use_flash_attn:
                # ``use_flash_attn: False``: scores, fp32 masked softmax and the value product as separate ops
                # (the reference's baddbmm + scale-mask-softmax + bmm path, transformer.py:492-592)
                # dropout of the attention probabilities under the model-parallel RNG, as transformer.py:489,556 of
                # the reference forks the tracker around its attention dropout
                with get_rng_tracker().fork():
                    o = ref.attention_varlen(q, k, v, meta.get("cu_seqlens"), True, None, slopes,
                                             self.args.attention_dropout if self.training else 0.0).reshape(T, nq)
            else:
                o = ops.flash_attention(q, k, v, meta.get("cu_seqlens"), meta.get("max_seqlen"), causal=True,
                                        alibi_slopes=slopes).reshape(T, nq)
        return self.o_proj(o)


class ParallelMLP(nn.Module):
    def __init__(self, args: ModelArgs):
        super().__init__()
        a = args
        self.act = a.glu_activation or "silu"
        f = a.intermediate_size
        self.gate_up = ColumnParallelLinear(a.hidden_size, sequence_parallel=a.sequence_parallel, sigma=a.init_sigma,
                                            dtype=a.params_dtype, segments=[("gate_proj", f), ("up_proj", f)])
        self.down_proj = RowParallelLinear(f, a.hidden_size, sequence_parallel=a.sequence_parallel,
                                           sigma=a.output_sigma(), dtype=a.params_dtype)
        self._register_state_dict_hook(_split_fused_hook("gate_up", None))
        self.register_load_state_dict_pre_hook(_merge_fused_hook(self.gate_up, "gate_up", None))

    def forward(self, x):
        return self.down_proj(ops.glu(self.gate_up(x), self.act))


def _split_fused_hook(fused_name, packed_name):
    """state_dict hook: expose the fused weight under the reference's per-projection names."""
    def hook(module, state, prefix, local_metadata):
        fused = getattr(module, fused_name)
        for kind in ("weight", "bias"):
            key = f"{prefix}{fused_name}.{kind}"
            if key not in state:
                continue
            t = state.pop(key)
            if packed_name is not None:
                state[f"{prefix}{packed_name}.{kind}"] = t
                continue
            off = 0
            for (name, _), n in zip(fused.segments, fused.local_sizes):
                state[f"{prefix}{name}.{kind}"] = t[off:off + n]
                off += n
        # adapters of the fused projection: <fused>.lora.<segment>.lora_X_weight -> <segment>.lora_X_weight
        lead = f"{prefix}{fused_name}.lora."
        for key in [k for k in state if k.startswith(lead)]:
            seg, leaf = key[len(lead):].split(".", 1)
            state[f"{prefix}{seg}.{leaf}"] = state.pop(key)
    return hook


def _merge_fused_hook(fused, fused_name, packed_name):
    def hook(module, state, prefix, *args):
        for kind in ("weight", "bias"):
            if packed_name is not None and f"{prefix}{packed_name}.{kind}" in state:
                state[f"{prefix}{fused_name}.{kind}"] = state.pop(f"{prefix}{packed_name}.{kind}")
                continue
            keys = [f"{prefix}{name}.{kind}" for name, _ in fused.segments]
            if all(k in state for k in keys):
                state[f"{prefix}{fused_name}.{kind}"] = torch.cat([state.pop(k) for k in keys], dim=0)
        for name, _ in fused.segments:
            for leaf in ("lora_A_weight", "lora_B_weight"):
                k = f"{prefix}{name}.{leaf}"
                if k in state:
                    state[f"{prefix}{fused_name}.lora.{name}.{leaf}"] = state.pop(k)
    return hook


class ParallelTransformerLayer(nn.Module):
    """Pre-norm block.  The residual add of each half is folded into the following norm
    kernel: the layer receives ``(delta, residual)`` — the stream is ``residual + delta`` —
    and returns the same pair, so an add never runs as its own kernel
    (llama/transformer.py:756-802 does two separate adds)."""

    def __init__(self, args: ModelArgs, layer_number):
        super().__init__()
        self.layer_number = layer_number
        self.input_layernorm = build_layer_norm(args)
        self.self_attn = ParallelAttention(args, layer_number)
        self.post_attention_layernorm = build_layer_norm(args)
        self.mlp = ParallelMLP(args)

    def forward(self, delta, residual, meta, kv_cache=None):
        if residual is None:
            h = delta
            n1 = self.input_layernorm(h)
        else:
            n1, h = self.input_layernorm(delta, residual)
        attn = self.self_attn(n1, meta, kv_cache)
        n2, h = self.post_attention_layernorm(attn, h)
        return self.mlp(n2), h


class Embedding(nn.Module):
    """Token (+ optional absolute position) embedding producing the token-major stream,
    scattered along tokens when sequence parallel."""

    def __init__(self, args: ModelArgs):
        super().__init__()
        a = args
        self.args = a
        self.word_embeddings = VocabParallelEmbedding(a.vocab_size, a.hidden_size, sigma=a.embed_init_sigma,
                                                      dtype=a.params_dtype)
        self.position_embeddings = None
        if a.position_embedding_type == "absolute":
            self.position_embeddings = nn.Embedding(a.max_position_embeddings, a.hidden_size, dtype=a.params_dtype,
                                                    device=_device())
            nn.init.normal_(self.position_embeddings.weight, 0.0, a.embed_init_sigma)
        self.dropout = a.hidden_dropout

    def forward(self, ids_flat, position_ids_flat):
        g = get_grid()
        emb = self.word_embeddings
        emb.check_ids(ids_flat)
        x = emb.lookup(ids_flat)
        if self.position_embeddings is not None:
            pe = self.position_embeddings(position_ids_flat)
            x = x + (pe / g.tp if g.tp > 1 else pe)
        if g.tp > 1:
            if self.args.sequence_parallel:
                x = mp.reduce_scatter_to_sequence_parallel_region(x)
            else:
                x = mp.reduce_from_tensor_model_parallel_region(x)
        if self.dropout and self.training:
            x = F.dropout(x, self.dropout)
        return x


class LMHead(nn.Module):
    """Untied output projection holding a vocab-parallel ``word_embeddings.weight``."""

    def __init__(self, args: ModelArgs):
        super().__init__()
        self.args = args
        self.word_embeddings = VocabParallelEmbedding(args.vocab_size, args.hidden_size, sigma=args.head_init_sigma,
                                                      dtype=args.params_dtype)

    def gathered_input(self, x):
        if self.args.sequence_parallel and get_grid().tp > 1:
            return mp.gather_from_sequence_parallel_region(x, True)
        return mp.copy_to_tensor_model_parallel_region(x) if get_grid().tp > 1 else x

    def forward(self, x):
        xin = self.gathered_input(x)
        logits = ops.linear(xin, self.word_embeddings.weight)
        if getattr(self, "lora_head", False):
            from .lora import head_lora_logits
            logits = logits + head_lora_logits(self, xin)
        if not self.args.parallel_output:
            logits = mp.gather_from_tensor_model_parallel_region(logits)
        return logits
