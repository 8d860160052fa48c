"""Logit transformations and sampling.

Order and edge cases of the reference (``astrai/inference/runtime/sample.py:18-386``): temperature (clamped to 1e-8)
-> top-k (per-row k, strictly-smaller-than-threshold removed, k <= 0 disables) -> top-p (sorted descending, a token is
removed when the cumulative mass BEFORE it already exceeds p, so the first crossing token stays) -> frequency penalty
(only when some penalty is non-zero).  All temperatures exactly 0 => argmax of the raw logits.  The returned log-prob is
taken from the post-filter distribution.  Everything stays on the device; the caller decides when to synchronise.
"""

from __future__ import annotations

from typing import List, Optional, Union

import torch
from torch import Tensor

Scalar = Union[float, int, Tensor]
NEG_INF = -float("inf")


def _col(value: Scalar, like: Tensor, dtype=None) -> Union[float, Tensor]:
    if isinstance(value, Tensor):
        return value.to(like.device, non_blocking=True).to(dtype or value.dtype).view(-1, 1)
    return value


class BaseSamplingStrategy:
    def apply(self, logits: Tensor, filter_value: float = NEG_INF, input_ids: Optional[Tensor] = None,
              input_mask: Optional[Tensor] = None) -> Tensor:
        raise NotImplementedError


class TemperatureStrategy(BaseSamplingStrategy):
    def __init__(self, temperature: Scalar = 1.0):
        self.temperature = temperature

    def apply(self, logits, filter_value=NEG_INF, input_ids=None, input_mask=None):
        t = _col(self.temperature, logits)
        if isinstance(t, Tensor):
            return logits / t.clamp(min=1e-8).to(logits.dtype)
        return logits if t == 1.0 else logits / max(t, 1e-8)


class TopKStrategy(BaseSamplingStrategy):
    def __init__(self, top_k: Scalar = 0, max_k: Optional[int] = None):
        self.top_k = top_k
        self.max_k = max_k  # host-side upper bound of a tensor-valued k: avoids a device read

    def apply(self, logits, filter_value=NEG_INF, input_ids=None, input_mask=None):
        k = self.top_k
        vocab = logits.size(-1)
        if isinstance(k, Tensor):
            k = k.to(logits.device, non_blocking=True).long().clamp(min=0)
            max_k = self.max_k if self.max_k is not None else int(k.max().item())
            if max_k <= 0:
                return logits
            max_k = min(max_k, vocab)
            top = torch.topk(logits, max_k, dim=-1).values
            idx = (k.clamp(max=max_k) - 1).clamp(min=0).view(-1, 1)
            thresh = top.gather(1, idx)
            thresh = torch.where((k > 0).view(-1, 1), thresh, torch.full_like(thresh, NEG_INF))
            return logits.masked_fill(logits < thresh, filter_value)
        if k > 0:
            thresh = torch.topk(logits, min(int(k), vocab), dim=-1).values[..., -1:]
            return logits.masked_fill(logits < thresh, filter_value)
        return logits


class TopPStrategy(BaseSamplingStrategy):
    def __init__(self, top_p: Scalar = 1.0, active: Optional[bool] = None):
        self.top_p = top_p
        self.active = active  # host-side knowledge of "some p < 1"

    def apply(self, logits, filter_value=NEG_INF, input_ids=None, input_mask=None):
        p = _col(self.top_p, logits)
        if isinstance(p, Tensor):
            active = self.active if self.active is not None else bool((p < 1.0).any())
        else:
            active = p < 1.0
        if not active:
            return logits
        sorted_logits, order = torch.sort(logits, descending=True, dim=-1)
        mass = torch.softmax(sorted_logits, dim=-1).cumsum(dim=-1)
        drop = mass > p
        drop = torch.cat([torch.zeros_like(drop[..., :1]), drop[..., :-1]], dim=-1)
        mask = torch.zeros_like(drop).scatter_(1, order, drop)
        return logits.masked_fill(mask, filter_value)


class FrequencyPenaltyStrategy(BaseSamplingStrategy):
    def __init__(self, penalty: Scalar = 0.0):
        self.penalty = penalty

    def apply(self, logits, filter_value=NEG_INF, input_ids=None, input_mask=None):
        if input_ids is None:
            return logits
        p = _col(self.penalty, logits, logits.dtype)
        if not isinstance(p, Tensor) and p == 0.0:
            return logits
        ids = input_ids.to(logits.device, non_blocking=True)
        weight = torch.ones_like(ids, dtype=logits.dtype)
        if input_mask is not None:
            weight = weight * input_mask.to(logits.device, non_blocking=True).to(logits.dtype)
        counts = torch.zeros_like(logits).scatter_add_(1, ids.clamp(min=0), weight)
        return logits - p * counts


class SamplingPipeline(BaseSamplingStrategy):
    def __init__(self, strategies: List[BaseSamplingStrategy], greedy: Optional[bool] = None):
        self.strategies = strategies
        self._greedy = greedy

    def apply(self, logits, filter_value=NEG_INF, input_ids=None, input_mask=None):
        for s in self.strategies:
            logits = s.apply(logits, filter_value, input_ids, input_mask)
        return logits

    def _is_greedy_pipeline(self) -> bool:
        if self._greedy is not None:
            return self._greedy
        if not self.strategies or not isinstance(self.strategies[0], TemperatureStrategy):
            return False
        t = self.strategies[0].temperature
        return bool((t == 0).all()) if isinstance(t, Tensor) else t == 0

    @torch.inference_mode()
    def sample(self, logits: Tensor, filter_value: float = NEG_INF, input_ids: Optional[Tensor] = None,
               input_mask: Optional[Tensor] = None, return_logprobs: bool = False, generator=None):
        if self._is_greedy_pipeline():
            tokens, dist = logits.argmax(dim=-1), logits
        else:
            dist = self.apply(logits.float(), filter_value, input_ids, input_mask)
            tokens = torch.multinomial(torch.softmax(dist, dim=-1), num_samples=1, generator=generator).squeeze(-1)
        if not return_logprobs:
            return tokens
        logp = torch.log_softmax(dist.float(), dim=-1).gather(-1, tokens.unsqueeze(-1)).squeeze(-1)
        return tokens, logp


# ---- fused device path (ops/csrc/sampling.cu): one launch per step instead of topk / sort / cumsum / scatter / multinomial
_RNG = {"seed": None, "offset": 0}


def manual_seed(seed: int):
    """Seed of the fused sampler's Philox stream (the torch path uses the ``generator`` argument instead)."""
    _RNG["seed"], _RNG["offset"] = int(seed) & 0x7FFFFFFFFFFFFFFF, 0


def _fused_ok(logits: Tensor) -> bool:
    if not (logits.is_cuda and logits.dim() == 2 and logits.dtype in (torch.float32, torch.bfloat16) and logits.stride(1) == 1):
        return False
    from astrai_b200.ops import native

    return native.is_available()


def _row_tensor(value: Scalar, rows: int, dtype, device) -> Tensor:
    if isinstance(value, Tensor):
        return value.to(device=device, dtype=dtype, non_blocking=True).reshape(-1).expand(rows).contiguous()
    return torch.full((rows,), value, dtype=dtype, device=device)


def _sample_fused(logits, temperature, top_k, top_p, frequency_penalty, input_ids, input_mask, return_logprobs, hints):
    rows, dev = logits.shape[0], logits.device
    if "greedy" in hints:
        greedy = bool(hints["greedy"])
    elif isinstance(temperature, Tensor):
        greedy = bool((temperature == 0).all())
    else:
        greedy = temperature == 0
    if "has_freq" in hints:
        has_freq = bool(hints["has_freq"])
    elif isinstance(frequency_penalty, Tensor):
        has_freq = bool((frequency_penalty != 0).any())
    else:
        has_freq = frequency_penalty != 0
    has_freq = has_freq and input_ids is not None
    if _RNG["seed"] is None:
        manual_seed(torch.initial_seed())
    _RNG["offset"] += 1
    hist = input_ids.to(dev, non_blocking=True).long().contiguous() if has_freq else None
    mask = input_mask.to(dev, non_blocking=True).bool().contiguous() if (has_freq and input_mask is not None) else None
    tokens, logp, _work = torch.ops.astrai_b200.sample_rows(
        logits, _row_tensor(temperature, rows, torch.float32, dev), _row_tensor(top_k, rows, torch.int32, dev),
        _row_tensor(top_p, rows, torch.float32, dev),
        _row_tensor(frequency_penalty, rows, torch.float32, dev) if has_freq else None, hist, mask, greedy, _RNG["seed"],
        _RNG["offset"])
    return (tokens, logp) if return_logprobs else tokens


@torch.inference_mode()
def sample(logits: Tensor, temperature: Scalar = 1.0, top_k: Scalar = 0, top_p: Scalar = 1.0,
           frequency_penalty: Scalar = 0.0, input_ids: Optional[Tensor] = None, input_mask: Optional[Tensor] = None,
           filter_value: float = NEG_INF, return_logprobs: bool = False, generator=None, hints: Optional[dict] = None):
    """One-call sampling.  ``hints`` may carry host-side facts (``max_k``, ``top_p_active``, ``has_freq``, ``greedy``)
    so that no device value has to be inspected."""
    hints = hints or {}
    if generator is None and filter_value == NEG_INF and _fused_ok(logits):
        return _sample_fused(logits, temperature, top_k, top_p, frequency_penalty, input_ids, input_mask, return_logprobs,
                             hints)
    if "has_freq" in hints:
        has_freq = hints["has_freq"]
    elif isinstance(frequency_penalty, Tensor):
        has_freq = bool((frequency_penalty != 0).any())
    else:
        has_freq = frequency_penalty != 0
    strategies: List[BaseSamplingStrategy] = [
        TemperatureStrategy(temperature), TopKStrategy(top_k, hints.get("max_k")), TopPStrategy(top_p, hints.get("top_p_active")),
    ]
    if has_freq:
        strategies.append(FrequencyPenaltyStrategy(frequency_penalty))
    return SamplingPipeline(strategies, hints.get("greedy")).sample(
        logits, filter_value=filter_value, input_ids=input_ids, input_mask=input_mask, return_logprobs=return_logprobs,
        generator=generator)
