"""Runner hooks on a stub runner: logger line and TFLOPs formula, early exit, auto-inserted logger (CPU)."""
import time
import types

import pytest
import torch


class _StubRunner:
    def __init__(self):
        from easyllm_b200.optim.microbatches import ConstantNumMicroBatches
        self.config = {"runtime": {"fp16": False}}
        self.model = types.SimpleNamespace(args=types.SimpleNamespace(
            num_layers=4, hidden_size=64, vocab_size=1000, glu_activation="silu", checkpoint_activations=False,
            dynamic_checkpoint=None))
        self.optimizer = types.SimpleNamespace(param_groups=[{"lr": 1e-4}])
        self.engine = types.SimpleNamespace(get_global_grad_norm=lambda: 1.25, optimizer=types.SimpleNamespace(cur_scale=1.0))
        self.micro_batch_size, self.seq_length = 2, 128
        self.num_microbatches_calculator = ConstantNumMicroBatches(global_batch_size=8, micro_batch_size=2)
        self.total_train_iters, self.consumed_train_samples, self.consumed_train_tokens = 10, 16, 2048
        self.start_time, self.device = time.time(), torch.device("cpu")
        self.saved = []

    def save_checkpoint(self, it):
        self.saved.append(it)


def test_model_flops_formula():
    from easyllm_b200.runners.hooks import model_flops_per_iteration
    b, s, L, h, V = 8, 4096, 32, 4096, 32000
    want = 32 * 3 * b * s * L * h * h * (1 + s / (6 * h) + V / (16 * L * h))
    assert model_flops_per_iteration(b, s, L, h, V, glu=True, recompute=False) == pytest.approx(want)
    assert model_flops_per_iteration(b, s, L, h, V, glu=False, recompute=True) == pytest.approx(want * 24 * 4 / (32 * 3))


def test_logger_line_and_auto_insertion():
    from easyllm_b200.runners.hooks import TrainValLoggerHook, build_hooks
    r = _StubRunner()
    hooks = build_hooks(r, [{"type": "empty_cache", "kwargs": {"freq": 1}}])     # a logger is added when none is configured
    logger = next(h for h in hooks._hooks if isinstance(h, TrainValLoggerHook))
    logger.writer = None
    hooks("before_train")
    hooks("after_train_iter", 0, {"lm_loss": torch.tensor(2.5)})
    line = logger.last_line
    for piece in ("iteration        1/      10", "consumed samples:", "learning rate: 1.000E-04", "global batch size:     8",
                  "lm_loss: 2.500000E+00", "grad norm: 1.250", "number of nan iterations:   0", "TFLOPs:", "ETA Time:"):
        assert piece in line, (piece, line)
    hooks("after_train_iter", 1, {"lm_loss": torch.tensor(float("nan"))})
    assert "number of nan iterations:   1" in logger.last_line


def test_early_exit_saves_then_exits():
    from easyllm_b200.runners.hooks import EarlyExitHook
    r = _StubRunner()
    h = EarlyExitHook(r, exit_interval=3)
    h.after_train_iter(0)
    h.after_train_iter(1)
    with pytest.raises(SystemExit):
        h.after_train_iter(2)
    assert r.saved == [3]
    r2 = _StubRunner()
    r2.start_time = time.time() - 3600
    with pytest.raises(SystemExit):
        EarlyExitHook(r2, exit_duration_in_mins=30).after_train_iter(6)
    assert r2.saved == [7]


def test_torch_profiler_hook_writes_a_trace_for_the_active_window(tmp_path):
    import json
    from easyllm_b200.runners.hooks import TorchProfilerHook, build_hooks
    r = _StubRunner()
    hooks = build_hooks(r, [{"type": "torch_profiler", "kwargs": {"out_dir": str(tmp_path), "wait": 1, "warmup": 1,
                                                                   "active": 2, "row_limit": 5}}],
                        add_log_if_not_exists=False)
    h = next(x for x in hooks._hooks if isinstance(x, TorchProfilerHook))
    hooks("before_train")
    a = torch.randn(64, 64)
    for it in range(5):
        (a @ a).sum().item()
        hooks("after_train_iter", it, {})
    hooks("after_train")
    assert len(h.written) == 1 and h.written[0].endswith("trace_rank0_iter3.json")     # iterations 2 and 3 recorded
    trace = json.load(open(h.written[0]))
    assert any("mm" in str(e.get("name", "")) for e in trace["traceEvents"])
    assert (tmp_path / "trace_rank0_iter3.txt").read_text().strip()
    # a rank outside `ranks` does nothing
    idle = TorchProfilerHook(r, out_dir=str(tmp_path / "x"), ranks=(3,))
    idle.before_train(); idle.after_train_iter(0); idle.after_train()
    assert idle.written == [] and not (tmp_path / "x").exists()
