"""Training losses (registry ``LOSS_REGISTRY``).

Parity: llm/models/mg_models/llama/losses.py:11-284 — ``softmax_cross_entropy`` (masked mean
over ``loss_mask ∧ labels≠-100``; prefix-LM normaliser variants), ``reward_sigmoid_entropy``
(pairwise reward-model loss), ``mini_rlhf_entropy`` (ranking + SFT on the best sample) and
``dpo_loss`` (sigmoid / hinge against offline reference log-probs, SFT fallback when the
reference log-prob slot carries a value > 1).

Every loss is computed from *vocab-parallel* quantities: label log-probabilities are
``-CE(logits, label)`` evaluated shard-wise and combined with three scalars per token, so
no rank ever materialises gathered ``[b, s, V]`` logits (the reference all-gathers them for
the RLHF / DPO losses).
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn.functional as F

from .. import ops
from ..config.registry import LOSS_REGISTRY
from ..parallel.grid import get_grid
from ..utils.log import default_logger as logger

IGNORE_INDEX = -100


def _safe_labels(labels):
    return labels.masked_fill(labels == IGNORE_INDEX, 0)


def label_logps(vocab_parallel_logits, labels, cut_size=None):
    """log p(label) per token from vocab-parallel logits; ignored positions give 0."""
    mask = labels != IGNORE_INDEX
    lp = -ops.vocab_parallel_cross_entropy(vocab_parallel_logits, _safe_labels(labels), cut_size)
    return lp * mask, mask


@LOSS_REGISTRY.register("softmax_cross_entropy")
class CrossEntropy:
    def __init__(self, loss_on_targets_only=False, reweight_loss_based_on_position_frequency=False,
                 is_prefix=True, cut_size=None, **kwargs):
        self.loss_on_targets_only = loss_on_targets_only
        self.reweight = reweight_loss_based_on_position_frequency
        self.is_prefix = is_prefix
        self.cut_size = cut_size

    def normaliser(self, labels, loss_mask):
        """(expected token count, effective mask [T])."""
        mask = loss_mask.reshape(-1).to(torch.float32) * (labels.reshape(-1) != IGNORE_INDEX)
        if not self.is_prefix:
            return mask.sum(), mask
        mb, s = labels.shape
        if self.loss_on_targets_only:
            if self.reweight:
                w = torch.arange(s, 0, -1, dtype=torch.float, device=mask.device) / (s + 1) * 2
                avg = w.flip(-1).cumsum(-1).mean()
            else:
                avg = (s + 1) / 2
        else:
            avg = s
        return avg * mb, mask

    def from_token_losses(self, losses, labels, loss_mask):
        n, mask = self.normaliser(labels, loss_mask)
        return torch.sum(losses.reshape(-1) * mask) / n

    def __call__(self, output, labels):
        labels, loss_mask = labels[0], labels[1]
        losses = ops.vocab_parallel_cross_entropy(output, _safe_labels(labels), self.cut_size)
        return self.from_token_losses(losses, labels, loss_mask)


@LOSS_REGISTRY.register("reward_sigmoid_entropy")
class RewardSigmoidCrossEntropy:
    """Pairwise reward loss: first half of the batch is *chosen*, second half *rejected*;
    ``-logsigmoid(r_c - r_r)`` averaged from the first diverging token to the longer end."""

    def __init__(self, **kwargs):
        pass

    def __call__(self, output, labels):
        ids = labels[0]
        rewards = output[..., 0]
        g = get_grid()
        if g.tp_rank == 0:
            bs, s = ids.shape[0] // 2, ids.shape[1]
            loss = output.new_zeros(())
            for i in range(bs):
                c_id, r_id = ids[i], ids[bs + i]
                c_rw, r_rw = rewards[i], rewards[bs + i]
                c_pad = (c_id == IGNORE_INDEX).nonzero()
                c_end = int(c_pad[0]) if len(c_pad) else s
                div = (c_id != r_id).nonzero()
                if len(div) == 0:
                    end, start = r_rw.size(-1), r_rw.size(-1) - 1
                else:
                    r_pad = (r_id == IGNORE_INDEX).nonzero()
                    r_end = int(r_pad[0]) if len(r_pad) else s
                    end, start = max(c_end, r_end), int(div[0])
                loss = loss + -F.logsigmoid(c_rw[start:end] - r_rw[start:end]).mean()
        else:
            loss = output.mean() * 0
        if g.tp > 1:
            dist.all_reduce(loss, group=g.tp_group)
        return loss


@LOSS_REGISTRY.register("mini_rlhf_entropy")
class MiniRLHFCrossEntropy(CrossEntropy):
    def __init__(self, rlhf_weight=1.0, length_penalty=1.0, sentense_pairs=6, **kwargs):
        super().__init__(**{k: v for k, v in kwargs.items() if k in ("is_prefix", "cut_size")})
        self.rlhf_weight, self.length_penalty, self.sentense_pairs = rlhf_weight, length_penalty, sentense_pairs

    def __call__(self, output, labels):
        lab, rw = labels[0], labels[2]
        lp, mask = label_logps(output, lab, self.cut_size)                      # [B, L]
        scores = lp.sum(-1) / (mask.float().sum(-1) ** self.length_penalty)
        scores = scores.reshape(-1, self.sentense_pairs)
        rw = rw.reshape(-1, self.sentense_pairs)
        diff = scores.unsqueeze(-2) - scores.unsqueeze(-1)
        rw_diff = rw.unsqueeze(-2) - rw.unsqueeze(-1)
        rlhf = -diff[(rw_diff > 0) & (diff < 0)].sum()
        best = torch.argmax(rw, dim=-1)
        pick = torch.zeros_like(rw, dtype=torch.bool)
        pick.scatter_(1, best.unsqueeze(-1), True)
        pick = pick.reshape(-1)
        sft = -(lp[pick] * mask[pick]).sum() / mask[pick].float().sum()
        return self.rlhf_weight * rlhf + sft


@LOSS_REGISTRY.register("dpo_loss")
class DPOLoss(CrossEntropy):
    def __init__(self, rlhf_weight=1.0, length_penalty=1.0, sentense_pairs=2, beta=0.1, loss_fn="sigmoid",
                 reference_free=False, **kwargs):
        super().__init__(**kwargs)
        self.sentense_pairs, self.beta, self.loss_fn, self.reference_free = sentense_pairs, beta, loss_fn, reference_free
        logger.warning_once("DPOLoss only support micro_batch_size set to 1 now.")
        if sentense_pairs != 2:
            logger.warning_once("DPOLoss only support sentense_pairs set to 2 now.")

    def pair_loss(self, pc, pr, rc, rr):
        logits = (pc - pr) - (0 if self.reference_free else (rc - rr))
        if self.loss_fn == "sigmoid":
            loss = -F.logsigmoid(self.beta * logits).sum()
        elif self.loss_fn == "hinge":
            loss = torch.relu(1 - self.beta * logits).sum()
        else:
            raise ValueError(f"Unknown loss type: {self.loss_fn}. Should be one of ['sigmoid', 'hinge']")
        return loss, self.beta * (pc - rc).detach(), self.beta * (pr - rr).detach()

    def __call__(self, output, labels):
        lab, loss_mask, ref = labels[0], labels[1], labels[2]
        if ref[0] > 1.0:  # no reference log-probs for this sample: plain SFT
            return CrossEntropy.__call__(self, output, (lab, loss_mask))
        lp, _ = label_logps(output, lab, self.cut_size)
        logps = lp.sum(-1).reshape(-1, self.sentense_pairs)
        ref = ref.reshape(-1, self.sentense_pairs)
        loss, _, _ = self.pair_loss(logps[:, 0], logps[:, 1], ref[:, 0], ref[:, 1])
        return loss
