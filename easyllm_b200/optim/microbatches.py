"""Number-of-micro-batches calculators (registry ``BATCH_CALCULATOR_REGISTRY``).

Parity: llm/utils/general/microbatches.py:43-145 and ``get_train_iters``
(llm/utils/general/utils.py:110-132).  ``constant_num``: global batch / (micro batch · DP).
``rampup_batch_size_num``: the global batch grows from ``start_batch_size`` by
``batch_size_increment`` every ``ramup_samples / n_increments`` consumed samples.
"""
from __future__ import annotations

from ..config.registry import BATCH_CALCULATOR_REGISTRY
from ..parallel.grid import get_grid
from ..utils.log import default_logger as logger


class NumMicroBatchesCalculator:
    num_micro_batches = None
    current_global_batch_size = None

    def get(self):
        return self.num_micro_batches

    def get_current_global_batch_size(self):
        return self.current_global_batch_size

    def update(self, consumed_samples, consistency_check):
        pass


@BATCH_CALCULATOR_REGISTRY.register("constant_num")
class ConstantNumMicroBatches(NumMicroBatchesCalculator):
    def __init__(self, global_batch_size, micro_batch_size):
        per_step = micro_batch_size * get_grid().dp
        if global_batch_size % per_step:
            raise ValueError(f"global batch size ({global_batch_size}) is not divisible by micro batch size "
                             f"({micro_batch_size}) times data parallel size ({get_grid().dp})")
        self.num_micro_batches = global_batch_size // per_step
        self.global_batch_size = self.current_global_batch_size = global_batch_size


@BATCH_CALCULATOR_REGISTRY.register("rampup_batch_size_num")
class RampupBatchsizeNumMicroBatches(NumMicroBatchesCalculator):
    def __init__(self, start_batch_size, batch_size_increment, ramup_samples, global_batch_size, micro_batch_size):
        self.micro_batch_size = micro_batch_size
        self.per_step = micro_batch_size * get_grid().dp
        if start_batch_size <= 0 or global_batch_size < start_batch_size or batch_size_increment <= 0:
            raise ValueError("need 0 < start_batch_size <= global_batch_size and a positive increment")
        span = global_batch_size - start_batch_size
        if span % batch_size_increment:
            raise ValueError(f"global batch size interval ({span}) is not divisible by the increment "
                             f"({batch_size_increment})")
        self.start_batch_size, self.global_batch_size = start_batch_size, global_batch_size
        self.batch_size_increment, self.ramup_samples = batch_size_increment, ramup_samples
        n_inc = span // batch_size_increment
        self.samples_per_increment = ramup_samples / n_inc if n_inc else float("inf")
        self.update(0, False)

    def update(self, consumed_samples, consistency_check):
        if consumed_samples > self.ramup_samples:
            self.current_global_batch_size = self.global_batch_size
        else:
            steps = int(consumed_samples / self.samples_per_increment)
            self.current_global_batch_size = min(self.start_batch_size + steps * self.batch_size_increment,
                                                 self.global_batch_size)
        if consistency_check and self.current_global_batch_size % self.per_step:
            raise ValueError(f"current global batch size ({self.current_global_batch_size}) is not divisible by "
                             f"micro-batch-size times data parallel size ({self.per_step})")
        self.num_micro_batches = self.current_global_batch_size // self.per_step


def build_num_microbatches_calculator(cfg):
    calc = BATCH_CALCULATOR_REGISTRY.build(cfg)
    if isinstance(calc, ConstantNumMicroBatches):
        logger.info(f"setting number of micro-batches to constant {calc.get()}")
    elif isinstance(calc, RampupBatchsizeNumMicroBatches):
        kw = cfg["kwargs"]
        logger.info(f"batch size rampup from {kw['start_batch_size']} to {kw['global_batch_size']} by "
                    f"{kw['batch_size_increment']} over {kw['ramup_samples']} samples")
    return calc


def get_train_iters(calculator, train_iters=None, train_samples=None):
    """Iterations needed to consume ``train_samples`` under a (possibly ramping) batch size."""
    if train_samples is None:
        return train_iters
    if isinstance(calculator, RampupBatchsizeNumMicroBatches):
        iters, consumed = 0, 0
        while consumed <= calculator.ramup_samples and consumed < train_samples:
            calculator.update(consumed, False)
            consumed += calculator.get_current_global_batch_size()
            iters += 1
        calculator.update(0, False)
        if consumed < train_samples:
            iters += (train_samples - consumed) // calculator.global_batch_size
        return iters
    return train_samples // calculator.get_current_global_batch_size()
