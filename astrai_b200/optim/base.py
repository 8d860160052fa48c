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


def _plain(method):
    return getattr(method, "__wrapped__", method)


class UntracedOptimizer(Optimizer):
    """``torch.optim.Optimizer`` without the guards against torch's tracing compiler.

    torch wraps ``add_param_group`` / ``zero_grad`` / ``state_dict`` / ``load_state_dict`` so that the compiler does not
    trace into them, and the first call through a wrapper imports the compiler (with its symbolic-algebra dependencies:
    several seconds in every process that builds an optimizer).  Nothing in this framework is traced, so the optimizers
    here call the plain functions the wrappers stand in front of."""

    def add_param_group(self, param_group):
        return _plain(Optimizer.add_param_group)(self, param_group)

    def zero_grad(self, set_to_none: bool = True):
        return _plain(Optimizer.zero_grad)(self, set_to_none)

    def state_dict(self):
        return _plain(Optimizer.state_dict)(self)

    def load_state_dict(self, state_dict):
        return _plain(Optimizer.load_state_dict)(self, state_dict)


def composite_step(sub_optimizers, closure=None):
    """One step of several optimizers that together stand for one: the closure runs once (with gradients enabled), before
    any of them steps; ``None`` entries are skipped."""
    loss = None
    if closure is not None:
        with torch.enable_grad():
            loss = closure()
    for sub in sub_optimizers:
        if sub is not None:
            sub.step()
    return loss


def composite_zero_grad(sub_optimizers, set_to_none: bool = True) -> None:
    for sub in sub_optimizers:
        if sub is not None:
            sub.zero_grad(set_to_none=set_to_none)


def composite_state_dict(named_sub_optimizers: Dict[str, Optional[Optimizer]]) -> dict:
    """``{name: state dict}`` with the empty slots kept as ``None`` (a model without matrices has no matrix optimizer)."""
    return {name: (sub.state_dict() if sub is not None else None) for name, sub in named_sub_optimizers.items()}


def refresh_param_groups(sub_optimizers) -> List[dict]:
    """The parameter groups of all parts, in order: what a learning-rate scheduler iterates over."""
    return [g for sub in sub_optimizers if sub is not None for g in sub.param_groups]


class CompositeOptimizer(UntracedOptimizer):
    """Routes disjoint parameter sets through named sub-optimizers; behaves as one optimizer."""

    def __init__(self, params, defaults: dict, subs: Dict[str, Optional[Optimizer]]):
        super().__init__(params, defaults)
        self._subs = subs
        self.param_groups = self._collect_groups()

    def _live(self) -> List[Optimizer]:
        return [s for s in self._subs.values() if s is not None]

    def _collect_groups(self):
        return refresh_param_groups(self._subs.values())

    @torch.no_grad()
    def step(self, closure=None):
        return composite_step(self._subs.values(), closure)

    def zero_grad(self, set_to_none: bool = True):
        composite_zero_grad(self._subs.values(), set_to_none)

    def state_dict(self) -> Dict[str, Any]:
        return composite_state_dict(self._subs)

    def load_state_dict(self, state_dict: Dict[str, Any]):
        missing = [n for n in self._subs if n not in state_dict]
        if missing:
            raise ValueError(f"Checkpoint optimizer state is not compatible with {type(self).__name__}: missing {missing}")
        for name, s in self._subs.items():
            if s is not None and state_dict[name] is not None:
                s.load_state_dict(state_dict[name])
        self.param_groups = self._collect_groups()
