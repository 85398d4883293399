"""``TorchOptimizerAdapter``: fp32 masters under low-precision parameters, loss scaling for fp16, and state that
survives a save / reload through the engine checkpoint on a pipeline- and a data-parallel layout."""
import os

import pytest
import torch

from dist_utils import run_ranks

TINY = dict(num_layers=2, hidden_size=128, num_attention_heads=4, intermediate_size=344, vocab_size=512,
            layer_norm_params={"kwargs": {"eps": 1e-5}}, checkpoint_activations=False)
SEQ, MBS = 64, 2


class _Probe(torch.nn.Module):
    """Least squares on a fixed batch: a loss whose trajectory shows every lost update."""

    def __init__(self, dtype):
        super().__init__()
        g = torch.Generator().manual_seed(0)
        self.w1 = torch.nn.Parameter((torch.randn(64, 32, generator=g) * 0.2).to(dtype))
        self.w2 = torch.nn.Parameter((torch.randn(32, 8, generator=g) * 0.2).to(dtype))
        self.x = torch.randn(256, 64, generator=g)
        self.y = torch.randn(256, 8, generator=g)

    def loss(self):
        h = torch.tanh(self.x.to(self.w1.dtype) @ self.w1)
        return ((h @ self.w2).float() - self.y).pow(2).mean()


def _run_probe(dtype, through_adapter, steps=200, lr=2e-5):
    from easyllm_b200.optim.torch_adapter import TorchOptimizerAdapter
    m = _Probe(dtype)
    inner = torch.optim.AdamW(m.parameters(), lr=lr, weight_decay=0.0)
    opt = TorchOptimizerAdapter(inner, m.named_parameters()) if through_adapter else inner
    losses = []
    for _ in range(steps):
        loss = m.loss()
        loss.backward()
        if through_adapter:
            opt.accumulate_grads()
        opt.step()
        if not through_adapter:
            inner.zero_grad()
        losses.append(float(loss))
    return losses, m


def test_bf16_parameters_follow_the_fp32_trajectory_for_200_steps():
    """At a fine-tuning learning rate most Adam updates are far below half a bf16 ulp of the weight.  With the
    adapter's fp32 masters the bf16 model loses as much loss as the fp32 one; the same optimizer applied to the bf16
    parameters directly stalls."""
    ref, _ = _run_probe(torch.float32, True)
    low, m = _run_probe(torch.bfloat16, True)
    naive, _ = _run_probe(torch.bfloat16, False)
    drop_ref, drop_low, drop_naive = ref[0] - ref[-1], low[0] - low[-1], naive[0] - naive[-1]
    assert drop_ref > 1e-3
    assert abs(drop_low - drop_ref) < 0.25 * drop_ref, (drop_ref, drop_low)
    assert drop_naive < 0.5 * drop_ref, (drop_ref, drop_naive)          # what the masters are there to prevent
    assert m.w1.dtype == torch.bfloat16                                   # the model itself stays in bf16


def test_fp16_overflow_skips_the_step_and_halves_the_scale():
    from easyllm_b200.optim.torch_adapter import TorchOptimizerAdapter
    m = _Probe(torch.float16)
    inner = torch.optim.SGD(m.parameters(), lr=1e-3)
    opt = TorchOptimizerAdapter(inner, m.named_parameters(), fp16=True,
                                loss_scale_cfg={"init_scale": 2.0 ** 10, "growth_interval": 2, "hysteresis": 1})
    before = [p.detach().clone() for p in m.parameters()]
    scale0 = opt.cur_scale
    (m.loss() * opt.cur_scale).backward()
    m.w1.grad[0, 0] = float("inf")
    opt.accumulate_grads()
    assert opt.step() is False and opt.skipped_steps == 1
    assert opt.cur_scale == scale0 / 2
    assert all(torch.equal(a, b) for a, b in zip(before, m.parameters()))
    assert all(float(p.main_grad.abs().sum()) == 0.0 for p in m.parameters())     # the bad gradients are gone
    # finite gradients: the step is taken with the unscaled gradient, and the scale grows back after the window
    ref = _Probe(torch.float32)
    with torch.no_grad():
        for p, q in zip(ref.parameters(), m.parameters()):
            p.copy_(q.float())
    ref_opt = torch.optim.SGD(ref.parameters(), lr=1e-3)
    for _ in range(2):
        (m.loss() * opt.cur_scale).backward()
        opt.accumulate_grads()
        assert opt.step() is True
        ref.loss().backward()
        ref_opt.step()
        ref_opt.zero_grad()
    assert opt.cur_scale == scale0
    for p, q in zip(ref.parameters(), m.parameters()):
        assert (p - q.float()).abs().max() < 2e-3 * p.abs().max()


def _engine(tp, pp, kind, seed=0):
    from easyllm_b200.parallel.grid import get_grid, initialize_model_parallel
    from easyllm_b200.models import llama_custom
    from easyllm_b200.optim.adam8bit import Adam8bit
    from easyllm_b200.optim.torch_adapter import TorchOptimizerAdapter
    from easyllm_b200.engine import PipelineEngine
    import torch.distributed as dist
    if dist.is_initialized():
        initialize_model_parallel(tp, pp)
    g = get_grid()
    torch.manual_seed(seed)
    model = llama_custom(**TINY)
    params = [p for p in model.parameters() if p.requires_grad]
    inner = Adam8bit(params, lr=1e-3, min_8bit_size=1024) if kind == "adam8bit" else torch.optim.Adam(params, lr=1e-3)
    opt = TorchOptimizerAdapter(inner, model.named_parameters(), grad_clip=1.0)
    eng = PipelineEngine(model, opt, None, {"train_micro_batch_size_per_gpu": MBS,
                                            "gradient_accumulation_steps": 4 // (MBS * g.dp)})
    return eng, opt


def _resume_case(rank, world, tp, pp, kind, out_dir):
    """Five steps straight through, against three steps + save + a fresh engine that loads + two steps."""
    from easyllm_b200.data.synthetic import synthetic_batches
    eng, _ = _engine(tp, pp, kind)
    it = synthetic_batches(TINY["vocab_size"], SEQ, MBS, seed=1)
    straight = [float(eng.train_batch(it)) for _ in range(5)]

    eng, _ = _engine(tp, pp, kind)
    it = synthetic_batches(TINY["vocab_size"], SEQ, MBS, seed=1)
    first = [float(eng.train_batch(it)) for _ in range(3)]
    eng.save_checkpoint(out_dir, client_state={"iteration": 3})
    eng2, opt2 = _engine(tp, pp, kind, seed=123)          # different initial weights: everything must come from disk
    eng2.load_checkpoint(out_dir)
    resumed = [float(eng2.train_batch(it)) for _ in range(2)]
    fresh, _ = _engine(tp, pp, kind, seed=123)
    fresh.load_checkpoint(out_dir, load_optimizer_states=False)
    it2 = synthetic_batches(TINY["vocab_size"], SEQ, MBS, seed=1)
    for _ in range(3 * (4 // MBS) // max(1, world // (tp * pp))):
        next(it2)
    cold = [float(fresh.train_batch(it2)) for _ in range(2)]
    return straight, first + resumed, cold, opt2.step_count


@pytest.mark.parametrize("tp,pp,kind", [(1, 2, "adam8bit"), (1, 1, "adam8bit"), (1, 2, "adam")])
def test_adapter_state_survives_save_and_reload(tmp_path, tp, pp, kind):
    """The wrapped optimizer's moments (8-bit blocks and scales included), its step count and the fp32 masters come
    back from the checkpoint: the resumed run repeats the uninterrupted one, while a run that reloads only the weights
    (fresh moments) visibly departs from it."""
    outs = run_ranks(2, _resume_case, tp, pp, kind, str(tmp_path / "ckpt"))
    for straight, resumed, cold, steps in outs:
        assert steps == 5
        assert max(abs(a - b) for a, b in zip(straight, resumed)) < 1e-5, (straight, resumed)
    straight, _, cold, _ = outs[-1]          # the last pipeline stage holds the loss
    assert abs(cold[-1] - straight[-1]) > 10 * max(abs(a - b) for a, b in zip(outs[-1][0], outs[-1][1])) + 1e-6
    assert os.path.exists(tmp_path / "ckpt" / "latest")
