"""Medusa speculative decoding: extra heads on a frozen base LM + tree-attention verification.

Parity: llm/models/hf_models/medusa/{medusa_model.py:38-413, utils.py:33-405, kv_cache.py,
medusa_choices.py}.  ``MedusaModel`` puts ``medusa_num_heads`` heads (``num_layers`` residual
SiLU blocks + a vocab projection initialised from the base LM head) on the final hidden states
of a frozen base model; head ``i`` is trained to predict token ``t + 2 + i`` (per-head CE and
top-1/3/5 accuracy).  ``medusa_generate`` drafts a token tree from the heads' top-k, verifies
all paths in one base-model pass with a tree attention mask over a static KV cache, accepts the
longest prefix by greedy match (temperature 0) or typical acceptance, and compacts the cache.

The tree is a ``MedusaTree`` built from a list of choice paths; named presets are generated
from (node budget, depth, top-k) by expanding paths in order of increasing rank sum rather
than shipped as literal tables.
"""
from __future__ import annotations

import heapq
import os
from types import SimpleNamespace

import torch
import torch.nn as nn
import torch.nn.functional as F

from ... import ops
from ...config.registry import MODULE_ZOO_REGISTRY
from .modeling import build_meta

IGNORE_TOKEN_ID = -100
TOPK = 10

_PRESETS = {"mc_sim_7b_63": (63, 4, 10), "mc_sim_7b_top5": (20, 4, 5), "mc_sim_7b_3_head_top5": (40, 3, 5)}


def build_choices(name_or_list, num_heads=None):
    """Named preset → list of paths (tuples of per-head ranks), most likely paths first."""
    if not isinstance(name_or_list, str):
        paths = [tuple(p) for p in name_or_list]
    else:
        budget, depth, topk = _PRESETS[name_or_list]
        depth = min(depth, num_heads or depth)
        heap, paths, seen = [(0, (0,))], [], set()
        while heap and len(paths) < budget:
            cost, path = heapq.heappop(heap)
            if path in seen:
                continue
            seen.add(path)
            paths.append(path)
            if path[-1] + 1 < topk:
                heapq.heappush(heap, (cost + 1, path[:-1] + (path[-1] + 1,)))
            if len(path) < depth:
                heapq.heappush(heap, (cost + 1 + len(path), path + (0,)))
    if num_heads is not None:
        paths = [p for p in paths if len(p) <= num_heads]
    have = set(paths)
    for p in list(paths):                      # every prefix of a path must be a node
        for k in range(1, len(p)):
            if p[:k] not in have:
                have.add(p[:k]); paths.append(p[:k])
    return sorted(have, key=lambda p: (len(p), p))


class MedusaTree:
    """Node 0 is the root (the token sampled from the base head); node i ≥ 1 is ``paths[i-1]``."""

    def __init__(self, paths, device):
        self.paths = paths
        n = len(paths) + 1
        index = {p: i + 1 for i, p in enumerate(paths)}
        mask = torch.eye(n, dtype=torch.bool)
        mask[:, 0] = True
        pos = torch.zeros(n, dtype=torch.long)
        tree_idx = torch.zeros(n, dtype=torch.long)
        for p, i in index.items():
            for k in range(1, len(p)):
                mask[i, index[p[:k]]] = True
            pos[i] = len(p)
            tree_idx[i] = p[-1] + TOPK * (len(p) - 1) + 1
        leaves = [p for p in paths if not any(q[:len(p)] == p and len(q) > len(p) for q in paths)]
        depth = max(len(p) for p in paths)
        retrieve = torch.full((len(leaves), depth + 1), -1, dtype=torch.long)
        for r, p in enumerate(sorted(leaves, key=lambda p: (-len(p), p))):
            retrieve[r, 0] = 0
            for k in range(1, len(p) + 1):
                retrieve[r, k] = index[p[:k]]
        self.attn_mask, self.position_ids = mask.to(device), pos.to(device)
        self.tree_indices, self.retrieve_indices = tree_idx.to(device), retrieve.to(device)
        self.size = n


class ResBlock(nn.Module):
    def __init__(self, hidden, dtype=None):
        super().__init__()
        self.linear = nn.Linear(hidden, hidden, dtype=dtype)
        nn.init.zeros_(self.linear.weight)          # starts as the identity map
        self.act = nn.SiLU()

    def forward(self, x):
        return x + self.act(self.linear(x))


class MedusaModel(nn.Module):
    def __init__(self, base_model, medusa_num_heads=4, medusa_num_layers=1, base_model_name_or_path=None, tokenizer=None):
        super().__init__()
        self.base_model = base_model
        self.config = base_model.config
        w = base_model.lm_head.weight
        self.hidden_size, self.vocab_size = w.shape[1], w.shape[0]
        self.medusa, self.medusa_num_layers = medusa_num_heads, medusa_num_layers
        self.base_model_name_or_path, self.tokenizer = base_model_name_or_path, tokenizer
        self.medusa_head = nn.ModuleList(
            nn.Sequential(*[ResBlock(self.hidden_size, w.dtype) for _ in range(medusa_num_layers)],
                          nn.Linear(self.hidden_size, self.vocab_size, bias=False, dtype=w.dtype))
            for _ in range(medusa_num_heads))
        self.medusa_head.to(w.device)
        for h in self.medusa_head:
            h[-1].weight.data.copy_(w.data)
        self._tree = None

    def get_tokenizer(self):
        return self.tokenizer

    @classmethod
    def from_pretrained(cls, medusa_head_name_or_path, base_model=None, medusa_num_heads=None, medusa_num_layers=None,
                        base_model_name_or_path=None, **kw):
        model = cls(base_model, medusa_num_heads, medusa_num_layers, base_model_name_or_path)
        if medusa_head_name_or_path:
            f = os.path.join(medusa_head_name_or_path, "medusa_lm_head.pth")
            if os.path.exists(f):
                model.medusa_head.load_state_dict(torch.load(f, map_location=w_device(base_model)), strict=True)
        return model

    def _hidden(self, input_ids, attention_mask=None, position_ids=None, caches=None, meta=None):
        meta = meta or build_meta(input_ids, attention_mask, position_ids)
        return self.base_model.hidden_states(input_ids, meta, caches)

    def forward(self, input_ids=None, attention_mask=None, labels=None, output_orig=False, position_ids=None,
                return_dict=None, **_):
        b, s = input_ids.shape
        with torch.no_grad():                       # the base model is frozen
            h = self._hidden(input_ids, attention_mask, position_ids).detach()
        logits = torch.stack([head(h).view(b, s, -1) for head in self.medusa_head], dim=0)
        if self.training and labels is not None:
            return self.compute_loss(logits, labels, return_dict)
        if output_orig:
            return logits, h.view(b, s, -1), ops.linear(h, self.base_model.head_weight()).view(b, s, -1)
        return logits

    def compute_loss(self, logits, labels, return_dict=False):
        out, total = {}, 0
        for i in range(self.medusa):
            lg = logits[i, :, :-(2 + i)].reshape(-1, logits.shape[-1]).float()
            lb = labels[..., 2 + i:].reshape(-1).to(lg.device)
            loss_i = F.cross_entropy(lg, lb, ignore_index=IGNORE_TOKEN_ID)
            total = total + loss_i
            keep = lb.ne(IGNORE_TOKEN_ID)
            for k in (1, 3, 5):
                top = lg.topk(k, dim=-1).indices[keep]
                out[f"medusa{i}_top{k}.accuracy"] = top.eq(lb[keep].unsqueeze(-1)).any(-1).float().mean()
            out[f"medusa{i}.loss"] = loss_i
        return SimpleNamespace(**out, keys=lambda: out.keys(), __getitem__=out.__getitem__, _d=out) if return_dict else total

    # ---- speculative decoding -----------------------------------------------------------------
    def _new_caches(self, batch, max_len):
        a = self.base_model.arch
        w = self.base_model.lm_head.weight
        return [{"k": torch.zeros(batch, max_len, a.kv_heads, a.head_dim, dtype=w.dtype, device=w.device),
                 "v": torch.zeros(batch, max_len, a.kv_heads, a.head_dim, dtype=w.dtype, device=w.device), "len": 0}
                for _ in range(a.num_hidden_layers)]

    def _step_logits(self, h):
        med = torch.stack([head(h) for head in self.medusa_head], 0).float()     # [heads, n, V]
        base = ops.linear(h, self.base_model.head_weight()).float()               # [n, V]
        return med, base

    @torch.no_grad()
    def medusa_generate(self, input_ids, medusa_generate=True, attention_mask=None, temperature=0.0, max_steps=512,
                        medusa_choices="mc_sim_7b_3_head_top5", posterior_threshold=0.09, posterior_alpha=0.3,
                        generate_mode="eval", eos_token_id=None, max_new_tokens=None):
        """Yields ``{'ids', 'new_tokens', 'accept_lengths'}`` after every verification step (batch 1)."""
        if input_ids.shape[0] != 1:
            raise ValueError("Only support batch size 1 for now!!")
        dev = input_ids.device
        eos = self.base_model.arch.eos_token_id if eos_token_id is None else eos_token_id
        paths = build_choices(medusa_choices, self.medusa)
        if self._tree is None or self._tree.paths != paths:
            self._tree = MedusaTree(paths, dev)
        tree = self._tree
        ids = input_ids.clone()
        budget = max_new_tokens or max_steps * (self.medusa + 1)
        caches = self._new_caches(1, ids.shape[1] + budget + tree.size + 8)
        h = self._hidden(ids, caches=caches)
        med, base = self._step_logits(h[-1:])
        accept_hist, new_tokens = [], 0
        for _ in range(max_steps):
            if not medusa_generate:
                nxt = base[-1].argmax().view(1, 1)
                ids = torch.cat((ids, nxt), 1)
                pos = torch.tensor([[ids.shape[1] - 1]], device=dev)
                h = self._hidden(nxt, position_ids=pos, caches=caches)
                med, base = self._step_logits(h[-1:])
                new_tokens += 1
                accept_hist.append(0)
            else:
                # draft: root = base argmax, then top-k of each head
                root = base[-1].argmax().view(1)
                cand_flat = torch.cat((root, med[:, -1].topk(TOPK, dim=-1).indices.reshape(-1)))
                tree_tokens = cand_flat[tree.tree_indices]                            # [n_tree]
                n0 = caches[0]["len"]
                pos = (tree.position_ids + n0).view(1, -1)
                meta = build_meta(tree_tokens.view(1, -1), None, pos)
                meta["tree_mask"] = tree.attn_mask
                h = self.base_model.hidden_states(tree_tokens.view(1, -1), meta, caches)
                med_t, base_t = self._step_logits(h)                                   # [heads, n_tree, V], [n_tree, V]
                ri = tree.retrieve_indices
                valid = ri >= 0
                rsafe = ri.clamp(min=0)
                cand = tree_tokens[rsafe]                                              # [paths, depth+1]
                logits = base_t[rsafe]                                                 # [paths, depth+1, V]
                best, acc = evaluate_posterior(logits, cand, valid, temperature, posterior_threshold, posterior_alpha)
                sel = rsafe[best, :acc + 1]                                            # accepted tree nodes
                ids = torch.cat((ids, tree_tokens[sel].view(1, -1)), 1)
                for c in caches:                                                       # compact accepted KV entries
                    c["k"][:, n0:n0 + acc + 1] = c["k"][:, n0 + sel]
                    c["v"][:, n0:n0 + acc + 1] = c["v"][:, n0 + sel]
                    c["len"] = n0 + acc + 1
                last = sel[-1]
                med, base = med_t[:, last:last + 1], base_t[last:last + 1]
                new_tokens += acc + 1
                accept_hist.append(int(acc))
            yield {"ids": ids, "new_tokens": new_tokens, "accept_lengths": accept_hist}
            tail = ids[0, input_ids.shape[1]:]
            if (eos is not None and bool((tail == eos).any())) or new_tokens >= budget:
                break


def w_device(model):
    return model.lm_head.weight.device


def evaluate_posterior(logits, candidates, valid, temperature, threshold, alpha):
    """Longest accepted prefix over candidate paths.  Greedy: the draft token must equal the
    argmax of the previous position; typical acceptance: p(token) > min(threshold, alpha·exp(−H))."""
    if temperature == 0:
        ok = (candidates[:, 1:] == logits[:, :-1].argmax(-1)) & valid[:, 1:]
    else:
        probs = torch.softmax(logits[:, :-1] / temperature, dim=-1)
        p_tok = probs.gather(-1, candidates[:, 1:].unsqueeze(-1)).squeeze(-1)
        ent = -(probs * torch.log(probs + 1e-5)).sum(-1)
        ok = (p_tok > torch.minimum(torch.full_like(ent, threshold), torch.exp(-ent) * alpha)) & valid[:, 1:]
    acc = torch.cumprod(ok.int(), dim=1).sum(1)
    a = int(acc.max())
    if a == 0:
        return 0, 0
    best = torch.nonzero(acc == a).flatten()
    if temperature == 0 or len(best) == 1:
        return int(best[0]), a
    ll = torch.log_softmax(logits[best, :a], -1).gather(-1, candidates[best, 1:a + 1].unsqueeze(-1)).sum((1, 2))
    return int(best[ll.argmax()]), a


@MODULE_ZOO_REGISTRY.register("medusa")
def build_medusa(**cfg):
    base_cfg = cfg.get("base_model")
    base = MODULE_ZOO_REGISTRY.build(base_cfg)
    return MedusaModel.from_pretrained(cfg.get("medusa_head_name_or_path"), base, cfg.get("medusa_num_heads", 3),
                                       cfg.get("medusa_num_layers", 1), (base_cfg.get("kwargs") or {}).get("model_name_or_path"))
