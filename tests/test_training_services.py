"""Learning-rate schedules, micro-batch calculators, loss scaling, SophiaG, Dynamic Checkpoint selection (CPU)."""
import math

import pytest
import torch


class _Opt:
    def __init__(self, lr=1.0):
        self.param_groups = [{"lr": lr}]


def test_iter_base_annealing_counts_samples():
    from easyllm_b200.optim.lr import IterBaseAnnealingLR
    opt = _Opt()
    # 10 iterations of 8 samples, 2 warm-up iterations: the schedule advances by the global batch
    s = IterBaseAnnealingLR(opt, max_lr=1e-3, min_lr=1e-4, decay_style="cosine", lr_decay_iters=10, global_batch_size=8,
                            lr_warmup_iters=2, use_checkpoint_lr_scheduler=False)
    assert opt.param_groups[0]["lr"] == 0.0
    s.step(8)
    assert opt.param_groups[0]["lr"] == pytest.approx(0.5e-3)
    s.step(8)
    assert opt.param_groups[0]["lr"] == pytest.approx(1e-3)
    s.step(8 * 4)                                          # half way through the decay
    ratio = (48 - 16) / (80 - 16)
    assert opt.param_groups[0]["lr"] == pytest.approx(1e-4 + 0.5 * (math.cos(math.pi * ratio) + 1) * 9e-4)
    s.step(8 * 10)
    assert opt.param_groups[0]["lr"] == pytest.approx(1e-4)
    # Megatron-compatible state: restored schedule continues at the same point
    sd = s.state_dict()
    assert {"max_lr", "warmup_steps", "num_steps", "decay_style", "decay_steps", "min_lr"} <= set(sd)
    with pytest.raises(ValueError):
        IterBaseAnnealingLR(_Opt(), 1e-3, 1e-4, "linear", lr_decay_iters=2, global_batch_size=4, lr_warmup_iters=2)


def test_sample_base_annealing_decays_on_tokens():
    from easyllm_b200.optim.lr import SampleBaseAnnealingLR
    opt = _Opt()
    s = SampleBaseAnnealingLR(opt, max_lr=2.0, min_lr=0.0, decay_style="linear", lr_decay_samples=100,
                              lr_warmup_samples=10, decay_tokens=1000, use_checkpoint_lr_scheduler=False)
    s.step(10, token_num=100)                              # end of warm-up: its token count is remembered
    assert opt.param_groups[0]["lr"] == pytest.approx(2.0) and s.warmup_tokens == 100
    s.step(10, token_num=550)
    assert opt.param_groups[0]["lr"] == pytest.approx(2.0 * (1 - 450 / 900))
    s.step(10, token_num=2000)
    assert opt.param_groups[0]["lr"] == 0.0


def test_hf_cosine():
    from easyllm_b200.optim.lr import HFCosineLR
    opt = _Opt(lr=4.0)
    s = HFCosineLR(opt, warmup_steps=2, training_steps=10)
    lrs = [opt.param_groups[0]["lr"]]
    for _ in range(10):
        s.step()
        lrs.append(opt.param_groups[0]["lr"])
    assert lrs[0] == 0.0 and lrs[1] == pytest.approx(2.0) and lrs[2] == pytest.approx(4.0)
    assert lrs[6] == pytest.approx(4.0 * 0.5 * (1 + math.cos(math.pi * 0.5))) and lrs[10] == pytest.approx(0.0, abs=1e-9)


def test_microbatch_calculators():
    from easyllm_b200.optim.microbatches import (ConstantNumMicroBatches, RampupBatchsizeNumMicroBatches,
                                                 get_train_iters)
    c = ConstantNumMicroBatches(global_batch_size=32, micro_batch_size=4)
    assert c.get() == 8 and c.get_current_global_batch_size() == 32
    assert get_train_iters(c, train_samples=320) == 10 and get_train_iters(c, train_iters=7) == 7
    r = RampupBatchsizeNumMicroBatches(start_batch_size=8, batch_size_increment=8, ramup_samples=48,
                                       global_batch_size=32, micro_batch_size=2)
    sizes = []
    for consumed in (0, 15, 16, 40, 48, 49, 1000):
        r.update(consumed, True)
        sizes.append(r.get_current_global_batch_size())
    assert sizes == [8, 8, 16, 24, 32, 32, 32] and r.get() == 16
    with pytest.raises(ValueError):
        RampupBatchsizeNumMicroBatches(8, 7, 48, 32, 2)
    # iterations to consume 200 samples: 8+8 (to 16), 16+16 (to 48), then 32 per step
    r.update(0, False)
    assert get_train_iters(r, train_samples=200) == 5 + (200 - 80) // 32


def test_dynamic_loss_scaler_hysteresis_and_growth():
    from easyllm_b200.optim.zero import DynamicLossScaler
    s = DynamicLossScaler(init_scale=1024.0, growth_interval=3, factor=2.0, min_scale=1.0, hysteresis=2)
    s.update(True)
    assert s.cur_scale == 1024.0                           # first overflow is absorbed by the hysteresis
    s.update(True)
    assert s.cur_scale == 512.0
    for _ in range(3):
        s.update(False)
    assert s.cur_scale == 1024.0
    t = DynamicLossScaler()
    t.load_state_dict(s.state_dict())
    assert t.cur_scale == 1024.0


def test_sophia_g_is_clipped_sign_momentum():
    from easyllm_b200.optim.sophia import SophiaG
    p = torch.nn.Parameter(torch.tensor([1.0, -2.0, 3.0]))
    opt = SophiaG([p], lr=0.1, betas=(0.0, 0.99), rho=0.04, weight_decay=0.0)
    p.grad = torch.tensor([0.5, -0.25, 0.0])
    opt.step(bs=1)
    # with a zero hessian estimate the update is lr * sign(momentum) (clipped at 1), zero gradient stays put
    assert torch.allclose(p.detach(), torch.tensor([0.9, -1.9, 3.0]), atol=1e-6)


def test_novograd_update_rule_and_builder_names():
    """Two hand-computed steps of the per-tensor second-moment rule; the builder resolves the apex names."""
    from easyllm_b200.optim import NovoGrad, build_optimizer
    p = torch.nn.Parameter(torch.tensor([3.0, 4.0]))
    opt = NovoGrad([p], lr=0.1, betas=(0.5, 0.5), eps=0.0, weight_decay=0.1, bias_correction=False)
    p.grad = torch.tensor([3.0, 4.0])
    opt.step()
    # v = |g|^2 = 25, u = g/5 + 0.1*w = [0.9, 1.2], m = 0.5*u, w -= 0.1*m
    w1 = torch.tensor([3.0 - 0.1 * 0.45, 4.0 - 0.1 * 0.6])
    assert torch.allclose(p.detach(), w1, atol=1e-6)
    p.grad = torch.tensor([0.0, 5.0])
    opt.step()
    # v = 0.5*25 + 0.5*25 = 25, u = [0, 1] + 0.1*w1, m = 0.5*[0.45, 0.6] + 0.5*u
    u2 = torch.tensor([0.0, 1.0]) + 0.1 * w1
    m2 = 0.5 * torch.tensor([0.45, 0.6]) + 0.5 * u2
    assert torch.allclose(p.detach(), w1 - 0.1 * m2, atol=1e-6)
    # bias correction divides the (un-decayed) first norm as well: denom = |g| / sqrt(1 - beta2) = 50
    q = torch.nn.Parameter(torch.tensor([3.0, 4.0]))
    o2 = NovoGrad([q], lr=0.1, betas=(0.9, 0.99), eps=0.0)
    q.grad = torch.tensor([3.0, 4.0])
    o2.step()
    # u = g/50; m = 0.1*u; m/c1 = u
    assert torch.allclose(q.detach(), torch.tensor([3.0 - 0.006, 4.0 - 0.008]), atol=1e-6)
    lin = torch.nn.Linear(4, 4)
    assert type(build_optimizer({"type": "FusedNovoGrad", "kwargs": {"lr": 0.1}}, lin)).__name__ == "NovoGrad"
    sgd = build_optimizer({"type": "FusedSGD", "kwargs": {"lr": 0.1, "momentum": 0.9, "weight_decay": 0.01}}, lin)
    assert isinstance(sgd, torch.optim.SGD) and sgd.param_groups[1]["weight_decay"] == 0.0
    with pytest.raises(RuntimeError):
        NovoGrad([q], amsgrad=True)


def test_adam8bit_tracks_fp32_adam_with_a_quarter_of_the_state():
    from easyllm_b200.optim import Adam8bit, build_optimizer
    from easyllm_b200.optim.adam8bit import (dequantize_signed, dequantize_unsigned, quantize_signed,
                                             quantize_unsigned)
    torch.manual_seed(0)
    x = torch.randn(5000) * torch.logspace(-4, 0, 5000)                 # four decades of magnitudes
    q, s = quantize_signed(x, 256)
    back = dequantize_signed(q, s, x.numel(), x.shape)
    assert q.dtype == torch.int8 and (back - x).abs().max() <= 0.02 * x.abs().max()
    big_enough = x.abs() > 1e-2
    assert torch.equal(torch.sign(back[big_enough]), torch.sign(x[big_enough]))
    v = x * x
    qv, sv = quantize_unsigned(v, 256)
    backv = dequantize_unsigned(qv, sv, v.numel(), v.shape)
    assert qv.dtype == torch.uint8 and (backv.sqrt() - v.sqrt()).abs().max() <= 0.02 * v.sqrt().max()

    def fit(make_opt):
        torch.manual_seed(1)
        net = torch.nn.Sequential(torch.nn.Linear(64, 128), torch.nn.Tanh(), torch.nn.Linear(128, 64))
        opt = make_opt(net)
        data = torch.randn(256, 64)
        target = data.roll(1, dims=1) * 0.5
        losses = []
        for _ in range(60):
            loss = ((net(data) - target) ** 2).mean()
            opt.zero_grad(); loss.backward(); opt.step()
            losses.append(loss.item())
        return losses, opt
    ref, _ = fit(lambda n: torch.optim.Adam(n.parameters(), lr=3e-3))
    got, opt8 = fit(lambda n: Adam8bit(n.parameters(), lr=3e-3, min_8bit_size=1024, block_size=256))
    assert got[-1] < 0.5 * got[0] and abs(got[-1] - ref[-1]) < 0.15 * ref[-1]
    # the two weight matrices (8192 elements each) hold 1 byte per moment, the biases keep fp32 state
    big = 2 * 8192
    assert opt8.state_bytes() < 2.3 * big + 8 * (128 + 64) + 4096
    lin = torch.nn.Linear(8, 8)
    assert type(build_optimizer({"type": "Adam8bit", "kwargs": {"lr": 1e-3}}, lin)).__name__ == "Adam8bit"
    assert build_optimizer({"type": "AdamW8bit", "kwargs": {"lr": 1e-3, "weight_decay": 0.1}}, lin).param_groups[0]["adamw"]


def test_dynamic_checkpoint_manager_selection():
    from easyllm_b200.utils.dc_manager import DynamicCheckpointManager, bfs_candidates

    class Block(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.lin = torch.nn.Linear(8, 8)

        def forward(self, x):
            return torch.relu(self.lin(x))

    class Net(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.embed = torch.nn.Embedding(16, 8)
            self.layers = torch.nn.ModuleList(Block() for _ in range(4))

        def forward(self, ids):
            x = self.embed(ids)
            for l in self.layers:
                x = l(x)
            return x.sum()

    net = Net()
    assert bfs_candidates(net) == [f"layers.{i}" for i in range(4)]
    dc = DynamicCheckpointManager(net, {128: 0, 512: 2, 1024: -1})
    assert dc.before_forward(torch.zeros(2, 100, dtype=torch.long)) == 0
    assert dc.before_forward(torch.zeros(2, 300, dtype=torch.long)) == 2 and dc.cur_checkpoint_modules == {"layers.0", "layers.1"}
    assert dc.before_forward(torch.zeros(1, 900, dtype=torch.long)) == 4           # -1: every candidate
    assert dc.before_forward(torch.zeros(1, 5000, dtype=torch.long)) == 4          # beyond the map: last key
    ids = torch.randint(0, 16, (2, 300))
    dc.before_forward(ids)
    a = net(ids); a.backward()
    g_ckpt = net.layers[0].lin.weight.grad.clone()
    net.zero_grad()
    dc.cur_checkpoint_modules = set()
    b = net(ids); b.backward()
    assert torch.allclose(a, b) and torch.allclose(g_ckpt, net.layers[0].lin.weight.grad)
