"""Failure detection without faulting any device: a rank that stops beating, a rank that exits,
graceful departure, NaN policies of the optimizer (skip / abort)."""
import time

import pytest
import torch

from dist_utils import run_ranks


def _beat(rank, world, port, mode):
    from easyllm_b200.parallel.watchdog import Watchdog, RankFailure
    wd = Watchdog(rank, world, port=port, interval=0.1, timeout=0.8).start()
    time.sleep(0.5)
    wd.check()                                   # everyone alive
    if mode == "hang" and rank == 1:
        wd.pause_heartbeat()                     # rank 1 stops beating but stays in the job
        time.sleep(3.0)
        wd.stop()
        return "hung"
    if mode == "leave" and rank == 1:
        wd.leave()                               # between steps, announced: not a failure
        return "left"
    deadline = time.time() + 3.0
    status = "ok"
    while time.time() < deadline:
        try:
            wd.check()
        except RankFailure as e:
            status = f"detected:{sorted(wd.failed_ranks)}"
            break
        time.sleep(0.1)
    wd.stop()
    return status


def _port():
    import socket
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close()
    return p


def test_hung_rank_is_detected():
    out = run_ranks(3, _beat, _port(), "hang")
    assert out[0] == "detected:[1]" and out[2] == "detected:[1]"


def test_graceful_leave_is_not_a_failure():
    out = run_ranks(2, _beat, _port(), "leave")
    assert out == ["ok", "left"]


def test_nan_policies():
    from easyllm_b200.optim import ZeroOptimizer
    lin = torch.nn.Linear(8, 8)
    opt = ZeroOptimizer(lin.named_parameters(), lr=0.1, stage=0, nan_policy="skip")
    before = lin.weight.detach().clone()
    lin.weight.main_grad.fill_(float("nan"))
    assert opt.step() is False and opt.skipped_steps == 1 and torch.equal(lin.weight, before)
    lin.weight.main_grad.fill_(1.0)
    assert opt.step() is True and not torch.equal(lin.weight, before)
    opt2 = ZeroOptimizer(torch.nn.Linear(4, 4).named_parameters(), lr=0.1, stage=0, nan_policy="abort")
    opt2.grad_buf.fill_(float("inf"))
    with pytest.raises(FloatingPointError):
        opt2.step()
