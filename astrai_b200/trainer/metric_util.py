"""Gradient statistics and the getters behind the names accepted by ``TrainConfig.metrics``.

Reference: ``astrai/trainer/metric_util.py:8-98``.  The SNR tracker walks the flat fp32 gradient buffers when the
model runs on the flat runtime (a handful of large tensors instead of one small tensor per parameter).
"""

from __future__ import annotations

import math
from typing import Dict, List, Union

import torch
import torch.nn as nn


def _grad_tensors(model: nn.Module) -> List[torch.Tensor]:
    engine = getattr(getattr(model, "module", model), "_flat_engine", None)
    if engine is not None:
        return [u.grad_buf for u in engine.units]
    return [p.grad.detach() for p in model.parameters() if p.grad is not None]


def grad_norm(model: nn.Module, per_param: bool = False) -> Union[float, Dict[str, float]]:
    grads = _grad_tensors(model)
    if not grads:
        return 0.0
    total = torch.stack([g.float().pow(2).sum() for g in grads]).sum().sqrt().item()
    if not per_param:
        return total
    out = {}
    for name, p in model.named_parameters():
        g = getattr(p, "main_grad", None)
        g = p.grad if g is None else g
        out[name] = g.float().norm(2).item() if g is not None else 0.0
    out["total"] = total
    return out


class GradSNRTracker:
    """EMA estimate of ``E[g]^2 / Var(g)`` over all gradient entries, reported in dB."""

    def __init__(self, beta: float = 0.999, eps: float = 1e-8):
        self.beta, self.eps = beta, eps
        self._first: Dict[int, torch.Tensor] = {}
        self._second: Dict[int, torch.Tensor] = {}

    @torch.no_grad()
    def update(self, model: nn.Module) -> None:
        for i, g in enumerate(_grad_tensors(model)):
            key = i
            if key not in self._first:
                self._first[key] = g.clone()
                self._second[key] = g * g
            else:
                self._first[key].mul_(self.beta).add_(g, alpha=1 - self.beta)
                self._second[key].mul_(self.beta).addcmul_(g, g, value=1 - self.beta)

    @property
    def snr(self) -> float:
        if not self._first:
            return 0.0
        signal = noise = 0.0
        for m, v in zip(self._first.values(), self._second.values()):
            m2 = m.float().pow(2)
            signal += m2.sum().item()
            noise += (v.float() - m2).clamp(min=0).sum().item()
        return 10.0 * math.log10(max(signal / (noise + self.eps), self.eps))


def ctx_get_loss(ctx):
    return ctx.loss


def ctx_get_lr(ctx):
    return ctx.optimizer.param_groups[-1]["lr"]


def ctx_get_val_loss(ctx):
    return ctx.val_loss


def ctx_get_grad_norm(ctx):
    return ctx.grad_norm


def ctx_get_grad_snr(ctx):
    tracker = getattr(ctx, "grad_snr_tracker", None)
    return None if tracker is None else tracker.snr


def ctx_get_moe_metric(ctx, key):
    return ctx.strategy._moe_metrics.get(key)
