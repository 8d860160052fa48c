"""Learning-rate schedules as multiplicative factors of the base rate.

Formulas of the reference (``astrai/trainer/schedule.py:59-74``, ``:116-145``, ``:195-208``).  All three share the
warm-up ``max(min_rate, step / max(warmup, 1))``; hyper-parameters travel inside ``state_dict``.
"""

from __future__ import annotations

import math
from typing import List

from torch.optim.lr_scheduler import LRScheduler

from astrai_b200.factory import BaseFactory


class BaseScheduler(LRScheduler):
    """Subclasses list their hyper-parameter names in ``_hparams`` and implement ``factor(step)``."""

    _hparams: tuple = ()

    def factor(self, step: int) -> float:
        raise NotImplementedError

    def warmup_factor(self, step: int) -> float:
        return max(self.min_rate, step / max(self.warmup_steps, 1))

    def get_lr(self) -> List[float]:
        f = self.factor(self.last_epoch)
        return [base * f for base in self.base_lrs]

    def state_dict(self):
        sd = super().state_dict()
        sd.update({k: getattr(self, k) for k in self._hparams})
        return sd

    def load_state_dict(self, state_dict):
        state_dict = dict(state_dict)
        for k in self._hparams:
            if k in state_dict:
                setattr(self, k, state_dict.pop(k))
        super().load_state_dict(state_dict)


class SchedulerFactory(BaseFactory["BaseScheduler"]):
    pass


@SchedulerFactory.register("cosine")
class CosineScheduler(BaseScheduler):
    _hparams = ("warmup_steps", "lr_decay_steps", "min_rate", "total_steps")

    def __init__(self, optimizer, warmup_steps: int, lr_decay_steps: int, min_rate: float = 0.01, last_epoch: int = -1):
        self.warmup_steps, self.lr_decay_steps, self.min_rate = warmup_steps, lr_decay_steps, min_rate
        self.total_steps = warmup_steps + lr_decay_steps
        super().__init__(optimizer, last_epoch)

    def factor(self, step):
        if step < self.warmup_steps:
            return self.warmup_factor(step)
        progress = min((step - self.warmup_steps) / max(self.lr_decay_steps, 1), 1.0)
        return max(self.min_rate, 0.5 * (1.0 + math.cos(math.pi * progress)))


@SchedulerFactory.register("sgdr")
class SGDRScheduler(BaseScheduler):
    _hparams = ("warmup_steps", "cycle_length", "min_rate", "t_mult")

    def __init__(self, optimizer, warmup_steps: int, cycle_length: int, min_rate: float = 0.01, t_mult: int = 2, last_epoch: int = -1):
        self.warmup_steps, self.cycle_length, self.min_rate, self.t_mult = warmup_steps, cycle_length, min_rate, t_mult
        super().__init__(optimizer, last_epoch)

    def factor(self, step):
        if step < self.warmup_steps:
            return self.warmup_factor(step)
        pos, length = step - self.warmup_steps, self.cycle_length
        while pos >= length:  # walk the restarts: each cycle is t_mult times longer
            pos -= length
            length *= self.t_mult
        return self.min_rate + (1 - self.min_rate) * 0.5 * (1 + math.cos(math.pi * pos / length))


@SchedulerFactory.register("wsd")
class WSDScheduler(BaseScheduler):
    """Warm-up, stable plateau at the base rate, then quadratic decay to ``min_rate``."""

    _hparams = ("warmup_steps", "stable_steps", "decay_steps", "min_rate", "total_steps")

    def __init__(self, optimizer, warmup_steps: int, stable_steps: int, decay_steps: int, min_rate: float = 0.01, last_epoch: int = -1):
        self.warmup_steps, self.stable_steps, self.decay_steps, self.min_rate = warmup_steps, stable_steps, decay_steps, min_rate
        self.total_steps = warmup_steps + stable_steps + decay_steps
        super().__init__(optimizer, last_epoch)

    def factor(self, step):
        if step < self.warmup_steps:
            return self.warmup_factor(step)
        off = step - self.warmup_steps
        if off < self.stable_steps:
            return 1.0
        ratio = min((off - self.stable_steps) / max(self.decay_steps, 1), 1.0)
        return (1.0 - self.min_rate) * (1.0 - ratio) ** 2 + self.min_rate
