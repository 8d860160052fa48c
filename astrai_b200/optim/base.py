"""Optimizer registry and helpers for optimizers composed of several sub-optimizers.

Reference: ``astrai/optim/composite.py:21-71``.
"""

from __future__ import annotations

from typing import Any, Dict, List, Optional

import torch
from torch.optim import Optimizer

from astrai_b200.factory import BaseFactory


class OptimizerFactory(BaseFactory[Optimizer]):
    """Built-in training optimizers by name."""


class CompositeOptimizer(Optimizer):
    """Routes disjoint parameter sets through named sub-optimizers; behaves as one optimizer."""

    def __init__(self, params, defaults: dict, subs: Dict[str, Optional[Optimizer]]):
        super().__init__(params, defaults)
        self._subs = subs
        self.param_groups = self._collect_groups()

    def _live(self) -> List[Optimizer]:
        return [s for s in self._subs.values() if s is not None]

    def _collect_groups(self):
        return [g for s in self._live() for g in s.param_groups]

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for s in self._live():
            s.step()
        return loss

    def zero_grad(self, set_to_none: bool = True):
        for s in self._live():
            s.zero_grad(set_to_none=set_to_none)

    def state_dict(self) -> Dict[str, Any]:
        return {name: (s.state_dict() if s is not None else None) for name, s in self._subs.items()}

    def load_state_dict(self, state_dict: Dict[str, Any]):
        missing = [n for n in self._subs if n not in state_dict]
        if missing:
            raise ValueError(f"Checkpoint optimizer state is not compatible with {type(self).__name__}: missing {missing}")
        for name, s in self._subs.items():
            if s is not None and state_dict[name] is not None:
                s.load_state_dict(state_dict[name])
        self.param_groups = self._collect_groups()
