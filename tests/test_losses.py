"""The four loss functions against direct restatements (CPU, world 1)."""
import math

import torch
import torch.nn.functional as F


def _logits(b, s, v, seed=0):
    return torch.randn(b, s, v, generator=torch.Generator().manual_seed(seed))


def test_softmax_cross_entropy_masked_mean():
    from easyllm_b200.models.losses import CrossEntropy
    out = _logits(2, 6, 11)
    labels = torch.randint(0, 11, (2, 6), generator=torch.Generator().manual_seed(1))
    labels[0, :2] = -100
    mask = torch.ones(2, 6, dtype=torch.long)
    mask[1, -1] = 0
    keep = (labels != -100) & (mask > 0)
    ref = F.cross_entropy(out.view(-1, 11), labels.clamp(min=0).view(-1), reduction="none").view(2, 6)
    # causal models (is_prefix False, what the model config expander selects): mean over the kept tokens
    loss = CrossEntropy(is_prefix=False)(out, (labels, mask))
    assert torch.allclose(loss, (ref * keep).sum() / keep.sum(), atol=1e-5)
    # prefix-LM normaliser: the expected token count b * s, whatever the mask
    loss_p = CrossEntropy(is_prefix=True)(out, (labels, mask))
    assert torch.allclose(loss_p, (ref * keep).sum() / 12, atol=1e-5)


def test_reward_pair_loss():
    from easyllm_b200.models.losses import RewardSigmoidCrossEntropy
    torch.manual_seed(0)
    ids = torch.tensor([[5, 6, 7, 8, -100, -100],       # chosen
                        [5, 6, 9, 9, 9, -100]])         # rejected: diverges at position 2, longer end at 5
    rewards = torch.randn(2, 6, 1)
    loss = RewardSigmoidCrossEntropy()(rewards, (ids,))
    want = -F.logsigmoid(rewards[0, 2:5, 0] - rewards[1, 2:5, 0]).mean()
    assert torch.allclose(loss, want, atol=1e-6)


def test_mini_rlhf_ranking_plus_sft():
    from easyllm_b200.models.losses import MiniRLHFCrossEntropy, label_logps
    out = _logits(4, 5, 9, seed=2)
    labels = torch.randint(0, 9, (4, 5), generator=torch.Generator().manual_seed(3))
    labels[:, 0] = -100
    rewards = torch.tensor([0.1, 0.9, 0.5, 0.2])
    fn = MiniRLHFCrossEntropy(rlhf_weight=2.0, length_penalty=1.0, sentense_pairs=4)
    loss = fn(out, (labels, torch.ones_like(labels), rewards))
    lp, mask = label_logps(out, labels)
    scores = lp.sum(-1) / mask.float().sum(-1)
    rank = 0.0
    for i in range(4):
        for j in range(4):
            if rewards[j] > rewards[i] and scores[j] < scores[i]:       # better sample scored lower: penalised
                rank += float(scores[i] - scores[j])
    best = int(rewards.argmax())
    sft = -(lp[best] * mask[best]).sum() / mask[best].float().sum()
    assert torch.allclose(loss, 2.0 * torch.tensor(rank) + sft, atol=1e-5)


def test_dpo_sigmoid_hinge_and_sft_fallback():
    from easyllm_b200.models.losses import CrossEntropy, DPOLoss, label_logps
    out = _logits(2, 5, 9, seed=4)
    labels = torch.randint(0, 9, (2, 5), generator=torch.Generator().manual_seed(5))
    mask = torch.ones_like(labels)
    ref = torch.tensor([-7.0, -9.0])
    lp, _ = label_logps(out, labels)
    pc, pr = lp[0].sum(), lp[1].sum()
    margin = (pc - pr) - (ref[0] - ref[1])
    sig = DPOLoss(beta=0.2, loss_fn="sigmoid")(out, (labels, mask, ref))
    assert torch.allclose(sig, -F.logsigmoid(0.2 * margin), atol=1e-5)
    hin = DPOLoss(beta=0.2, loss_fn="hinge")(out, (labels, mask, ref))
    assert torch.allclose(hin, torch.relu(1 - 0.2 * margin), atol=1e-5)
    free = DPOLoss(beta=0.2, reference_free=True)(out, (labels, mask, ref))
    assert torch.allclose(free, -F.logsigmoid(0.2 * (pc - pr)), atol=1e-5)
    # reference log-prob > 1 marks "no reference": the sample is trained as plain SFT
    sft = DPOLoss()(out, (labels, mask, torch.tensor([2.0, 2.0])))
    assert torch.allclose(sft, CrossEntropy()(out, (labels, mask)), atol=1e-6)
    assert math.isfinite(float(sft))
