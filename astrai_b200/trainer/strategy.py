"""Training objectives: next-token (seq), masked SFT, DPO and GRPO (offline and online).

Loss definitions are the reference's (``astrai/trainer/strategy.py:312-665``).  Two things differ by design:

* the vocabulary projection is fused with the loss (``ops.linear_cross_entropy`` / ``ops.linear_token_logprobs``)
  whenever the model can return hidden states without logits, so no ``[B*S, V]`` fp32 tensor is ever stored;
* metric values stay on the device until somebody reads them (:class:`DeferredMetrics`), which removes the
  reference's device->host sync on every micro-batch (``strategy.py:219-222``, ``trainer.py:86``).
"""

from __future__ import annotations

from typing import TYPE_CHECKING, Callable, Dict, List, Optional, TypedDict, Union

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch import Tensor

from astrai_b200 import ops
from astrai_b200.factory import BaseFactory
from astrai_b200.ops.segments import AttentionSegments, from_position_ids, from_valid_mask
from astrai_b200.parallel.executor import broadcast_state_dict

if TYPE_CHECKING:
    from astrai_b200.trainer.rollout import RolloutResult


class DeferredMetrics(dict):
    """A dict of scalars whose tensor values turn into Python floats only when read."""

    @staticmethod
    def _value(v):
        return float(v.detach().float().item()) if isinstance(v, Tensor) else v

    def __getitem__(self, key):
        v = self._value(dict.__getitem__(self, key))
        dict.__setitem__(self, key, v)
        return v

    def get(self, key, default=None):
        return self[key] if key in self else default

    def items(self):
        return [(k, self[k]) for k in dict.keys(self)]

    def values(self):
        return [self[k] for k in dict.keys(self)]

    def resolved(self) -> Dict[str, float]:
        return dict(self.items())


class LossOutput(TypedDict):
    loss: Tensor
    metrics: Dict[str, float]


class LogprobsOutput(TypedDict):
    logprobs: Tensor
    aux_loss: Optional[Tensor]
    router_stats: Optional[list]


def move_to_device(batch: Dict[str, Tensor], device) -> Dict[str, Tensor]:
    return {k: (v.to(device, non_blocking=True) if isinstance(v, Tensor) else v) for k, v in batch.items()}


def _fused_head(model) -> Optional[nn.Module]:
    """The module whose ``lm_head`` can be fused with the loss, or None (wrapped or foreign models)."""
    inner = getattr(model, "module", model)
    if getattr(inner, "supports_fused_head", False) and hasattr(inner, "lm_head"):
        return inner
    return None


def _head_weight(inner) -> Tensor:
    """``lm_head.weight`` for a fused projection + loss.  The ``lm_head`` module itself is not called on that path, so its
    forward pre-hook (where a sharded executor waits for the parameter's all-gather) never fires: ask the executor."""
    w = inner.lm_head.weight
    ex = getattr(inner, "_flat_executor", None)
    if ex is not None:
        ex.before_param_use(w)
    return w


def _token_logprobs_tensor_parallel(model, inner, input_ids: Tensor, input_mask):
    """The same ``[B, S-1]`` log-probabilities from a tensor-parallel model: every rank scores its own token rows of the
    whole ``[B, S]`` input (the target of a position is the next token; the last position of a row has none) and the
    per-token values are gathered, so that sequence-level objectives see whole sequences on every rank."""
    from astrai_b200.parallel.tensor_parallel import gather_row_values

    b, s = input_ids.shape
    tp, rank = inner._tp_size, inner._tp_rank
    local = b * s // tp
    targets = torch.cat([input_ids[:, 1:], input_ids.new_zeros(b, 1)], dim=1).reshape(-1)[rank * local:(rank + 1) * local]
    if getattr(inner, "supports_fused_head", False) and input_ids.is_cuda:
        out = model(input_ids, input_mask, return_logits=False)
        lp = ops.linear_token_logprobs(out["hidden_states"], _head_weight(inner), targets)
    else:
        out = model(input_ids, input_mask)
        lp = torch.log_softmax(out["logits"].float(), dim=-1).gather(-1, targets.unsqueeze(-1)).squeeze(-1)
    return gather_row_values(lp).view(b, s)[:, :-1], out


def token_logprobs(model, input_ids: Tensor, input_mask: Optional[Tensor], position_ids: Optional[Tensor] = None):
    """Log-probability of ``input_ids[:, 1:]`` under the model, shape ``[B, S-1]`` fp32, plus the forward outputs."""
    sharded = getattr(model, "module", model)
    if getattr(sharded, "_tp_size", 1) > 1:
        return _token_logprobs_tensor_parallel(model, sharded, input_ids, input_mask)
    ids_in, ids_out = input_ids[:, :-1], input_ids[:, 1:]
    if isinstance(input_mask, AttentionSegments):
        input_mask = input_mask.drop_last()
    elif input_mask is not None:
        input_mask = input_mask[:, :, :-1, :-1] if input_mask.dim() == 4 else input_mask[:, :-1]
    inner = _fused_head(model)
    if inner is not None and ids_in.is_cuda:
        out = model(ids_in, input_mask, return_logits=False)
        lp = ops.linear_token_logprobs(out["hidden_states"], _head_weight(inner), ids_out)
    else:
        out = model(ids_in, input_mask)
        lp = torch.log_softmax(out["logits"].float(), dim=-1).gather(-1, ids_out.unsqueeze(-1)).squeeze(-1)
    return lp, out


def reduce_logprobs(lp: Tensor, loss_mask: Tensor, reduction: str) -> Tensor:
    """``lp [B, S-1]`` masked by ``loss_mask[:, 1:]`` and summed / averaged per sequence, or left per token."""
    if reduction not in ("mean", "sum", "none"):
        raise ValueError(f"reduction must be one of ['mean', 'sum', 'none'], got '{reduction}'")
    m = loss_mask[:, 1:].to(lp.dtype)
    if reduction == "sum":
        return (lp * m).sum(-1)
    if reduction == "mean":
        return (lp * m).sum(-1) / m.sum(-1).clamp(min=1.0)
    return lp * m


def get_logprobs(model, input_ids: Tensor, attn_mask: Tensor, loss_mask: Tensor, reduction: str) -> LogprobsOutput:
    """Masked (and optionally reduced) next-token log-probabilities (reference ``strategy.py:33-84``)."""
    if reduction not in ("mean", "sum", "none"):
        raise ValueError(f"reduction must be one of ['mean', 'sum', 'none'], got '{reduction}'")
    lp, out = token_logprobs(model, input_ids, attn_mask)
    return {"logprobs": reduce_logprobs(lp, loss_mask, reduction), "aux_loss": out.get("aux_loss"), "router_stats": out.get("router_stats")}


def logprobs_from_logits(logits: Tensor, input_ids: Tensor) -> Tensor:
    """``[B, S-1]`` log-probability of ``input_ids[:, 1:]`` from logits of ALL ``S`` positions (the last one predicts nothing)."""
    return torch.log_softmax(logits[:, :-1].float(), dim=-1).gather(-1, input_ids[:, 1:].unsqueeze(-1)).squeeze(-1)


def dpo_loss(policy: Tensor, reference: Tensor, beta: float) -> Tensor:
    """``policy`` / ``reference`` ``[2n]``: sequence log-probabilities of ``n`` chosen answers, then of the ``n`` rejected ones."""
    n = policy.shape[0] // 2
    margin = (policy[:n] - policy[n:]) - (reference[:n] - reference[n:])
    return -F.logsigmoid(beta * margin).mean()


def grpo_terms(lp_pol: Tensor, lp_old: Tensor, lp_ref: Tensor, rewards: Tensor, tok: Tensor, clip_eps: float):
    """Sums over the response tokens ``tok [b, g, L]`` of the clipped surrogate and of the k3 KL estimate (not yet divided
    by a token count, not yet weighted): the two numerators of the GRPO loss."""
    eps = 1e-8
    adv = ((rewards - rewards.mean(-1, keepdim=True)) / (rewards.std(-1, keepdim=True, unbiased=False) + eps))[..., None]
    ratio = torch.exp(lp_pol - lp_old)
    surrogate = -torch.min(ratio * adv, ratio.clamp(1 - clip_eps, 1 + clip_eps) * adv)
    r = torch.exp(lp_ref - lp_pol)
    return (surrogate * tok).sum(), ((r - torch.log(r + eps) - 1.0) * tok).sum()


def make_doc_boundary_mask(position_ids: Tensor) -> Tensor:
    """``[B,1,S,S]`` bool: causal and within one packed document (a document starts where positions do not grow)."""
    b, s = position_ids.shape
    starts = position_ids[:, 1:] <= position_ids[:, :-1]
    doc = F.pad(starts.long().cumsum(dim=1), (1, 0))
    same = doc[:, :, None] == doc[:, None, :]
    causal = torch.ones(s, s, dtype=torch.bool, device=position_ids.device).tril()
    return (same & causal)[:, None]


def causal_padding_mask(key_valid: Tensor) -> Tensor:
    """``[B,1,S,S]`` bool: causal AND key is a real token."""
    s = key_valid.shape[-1]
    causal = torch.ones(s, s, dtype=torch.bool, device=key_valid.device).tril()
    return key_valid.bool()[:, None, None, :] & causal[None, None]


def doc_attention(position_ids: Tensor):
    """Attention restriction of a packed SFT batch: run boundaries for the variable-length flash kernels (no O(S^2)
    mask); the dense mask of :func:`make_doc_boundary_mask` is the same relation."""
    return from_position_ids(position_ids)


def padded_causal_attention(key_valid: Tensor):
    """Attention restriction of a padded batch (DPO / GRPO): run boundaries when every row's real tokens are contiguous
    (left and / or right padding), else the dense mask of :func:`causal_padding_mask` (padding inside a row)."""
    seg = from_valid_mask(key_valid)
    return seg if seg is not None else causal_padding_mask(key_valid)


def moe_diagnostics(router_stats_list) -> Dict[str, Tensor]:
    """Router entropy, dead-expert fraction and load imbalance (mean / max), averaged over MoE layers; device tensors."""
    rows: List[Tensor] = []
    for stats in router_stats_list or ():
        probs = stats["probs"].float()
        e = probs.shape[-1]
        probs = probs.reshape(-1, e)
        if e == 0 or probs.numel() == 0:
            continue
        idx = stats["topk_indices"].reshape(-1)
        entropy = -(probs * probs.clamp_min(1e-8).log()).sum(-1).mean()
        counts = torch.zeros(e, dtype=torch.float32, device=probs.device).scatter_add_(
            0, idx, torch.ones_like(idx, dtype=torch.float32))
        ratios = counts / counts.mean().clamp(min=1.0)
        rows.append(torch.stack([entropy, (counts == 0).float().mean(), (ratios - 1).abs().mean(), ratios.max()]))
    if not rows:
        return {}
    avg = torch.stack(rows).mean(0)
    names = ("router_entropy", "dead_expert_fraction", "load_imbalance_mean", "load_imbalance_max")
    return {n: avg[i] for i, n in enumerate(names)}


class BaseStrategy:
    """Turns a batch into ``{"loss": tensor, "metrics": {...}}``; online mode when a rollout runner is injected."""

    def __init__(self, model: Union[nn.Module, Callable[..., Dict[str, Tensor]]], device, **kwargs):
        self.model, self.device = model, device
        self.executor = kwargs.pop("executor", None)
        self.moe_aux_loss_coef = kwargs.pop("moe_aux_loss_coef", 0.01)
        self.strategy_kwargs = kwargs
        self._moe_metrics: Dict[str, float] = DeferredMetrics()
        self._rollout_runner = None

    def compute_loss(self, batch) -> Tensor:
        return self.compute_loss_output(batch)["loss"]

    def _to_rank(self, batch: Dict[str, Tensor]) -> Dict[str, Tensor]:
        """The batch on this rank's device, cut to this rank's share when the executor shards tokens (tensor / context
        parallelism); data-parallel executors leave it whole."""
        batch = move_to_device(batch, self.device)
        shard = getattr(self.executor, "shard_batch", None)
        return shard(batch) if shard is not None else batch

    def _whole_sequences(self, batch: Dict[str, Tensor]) -> Dict[str, Tensor]:
        """A sequence-level batch as the executor needs it laid out (a tensor-parallel block pads the sequences so that the
        batch's tokens divide over its ranks); other executors leave it alone."""
        pad = getattr(self.executor, "pad_sequences", None)
        return pad(batch) if pad is not None else batch

    def compute_loss_output(self, batch) -> LossOutput:
        out = self.compute_loss(batch)
        return out if isinstance(out, dict) else {"loss": out, "metrics": DeferredMetrics(loss=out.detach())}

    def _loss_output(self, task_loss: Tensor, metrics: Dict[str, Tensor], aux_loss: Optional[Tensor] = None,
                     router_stats=None) -> LossOutput:
        total = task_loss
        if aux_loss is not None:
            weighted = self.moe_aux_loss_coef * aux_loss
            total = total + weighted
            metrics["moe_aux_loss"], metrics["moe_aux_loss_weighted"] = aux_loss, weighted
            diag = DeferredMetrics(moe_diagnostics(router_stats))
            diag["aux_loss"] = aux_loss.detach()
            self._moe_metrics = diag
        metrics["loss"] = total
        return {"loss": total, "metrics": DeferredMetrics({k: (v.detach() if isinstance(v, Tensor) else v) for k, v in metrics.items()})}

    def supports_online(self) -> bool:
        return False

    def set_rollout_runner(self, runner):
        self._rollout_runner = runner

    def prepare_from_rollout(self, result: "RolloutResult") -> Dict[str, Tensor]:
        raise NotImplementedError(f"{type(self).__name__} does not support online rollout")

    def _on_rollout_refresh(self):
        pass

    def on_optimizer_step(self):
        if self._rollout_runner is not None:
            self._rollout_runner.step()

    def __call__(self, batch) -> LossOutput:
        if self._rollout_runner is None:
            return self.compute_loss_output(batch)
        result, fresh = self._rollout_runner(batch)
        if fresh:
            self._on_rollout_refresh()
        return self.compute_loss_output(self.prepare_from_rollout(result))


class StrategyFactory(BaseFactory["BaseStrategy"]):
    pass


class _TokenCEStrategy(BaseStrategy):
    def __init__(self, model, device, label_smoothing: float = 0.0, **kwargs):
        super().__init__(model, device, **kwargs)
        self.label_smoothing = label_smoothing

    def _ce(self, input_ids, targets, ignore_index=-100, **fwd):
        inner = _fused_head(self.model)
        if inner is not None and input_ids.is_cuda:
            out = self.model(input_ids=input_ids, return_logits=False, **fwd)
            loss = ops.linear_cross_entropy(out["hidden_states"], _head_weight(inner), targets,
                                            self.label_smoothing, ignore_index)
        else:
            out = self.model(input_ids=input_ids, **fwd)
            loss = ops.cross_entropy(out["logits"], targets, self.label_smoothing, ignore_index)
        return self._loss_output(loss, {"task_loss": loss}, out.get("aux_loss"), out.get("router_stats"))


@StrategyFactory.register("seq")
class SEQStrategy(_TokenCEStrategy):
    """Next-token cross-entropy over every position (mean), optional label smoothing."""

    def compute_loss_output(self, batch) -> LossOutput:
        batch = self._to_rank(batch)
        fwd = {"position_ids": batch["position_ids"]} if "position_ids" in batch else {}
        return self._ce(batch["input_ids"], batch["target_ids"], **fwd)


@StrategyFactory.register("sft")
class SFTStrategy(_TokenCEStrategy):
    """Cross-entropy on positions where ``loss_mask`` is set; attention stays inside each packed document."""

    def compute_loss_output(self, batch) -> LossOutput:
        attn = doc_attention(batch["position_ids"])  # from the host copy of the batch: no device round trip
        batch = self._to_rank(batch)
        pos = batch["position_ids"]
        targets = batch["target_ids"].masked_fill(~batch["loss_mask"].bool(), -100)
        # ranks that hold slices of one batch's tokens divide by their share of ALL trained tokens, not by their own count
        with ops.loss_denominator(batch.get("loss_denominator")):
            return self._ce(batch["input_ids"], targets, position_ids=pos, input_mask=attn)


@StrategyFactory.register("dpo")
class DPOStrategy(BaseStrategy):
    """``-logsigmoid(beta * ((pi_c - pi_r) - (ref_c - ref_r)))``; token id 0 is padding."""

    def __init__(self, model, device, ref_model, beta: float = 0.1, reduction: str = "sum", **kwargs):
        super().__init__(model, device, **kwargs)
        self.ref_model, self.beta, self.reduction = ref_model, beta, reduction

    def compute_loss_output(self, batch) -> LossOutput:
        batch = self._whole_sequences(batch)
        mask = padded_causal_attention(torch.cat([batch["chosen"], batch["rejected"]], dim=0).ne(0))
        batch = self._to_rank(batch)
        n = batch["chosen"].shape[0]
        ids = torch.cat([batch["chosen"], batch["rejected"]], dim=0)
        loss_mask = torch.cat([batch["chosen_mask"], batch["rejected_mask"]], dim=0)
        if isinstance(mask, Tensor):
            mask = mask.to(ids.device)
        pol = get_logprobs(self.model, ids, mask, loss_mask, self.reduction)
        with torch.no_grad():
            ref = get_logprobs(self.ref_model, ids, mask, loss_mask, self.reduction)["logprobs"]
        loss = dpo_loss(pol["logprobs"], ref, self.beta)
        return self._loss_output(loss, {"dpo_loss": loss}, pol["aux_loss"], pol.get("router_stats"))

    def supports_online(self) -> bool:
        return True

    def prepare_from_rollout(self, result: "RolloutResult") -> Dict[str, Tensor]:
        rows = torch.arange(result.responses.shape[0], device=result.responses.device)
        best, worst = result.rewards.argmax(-1), result.rewards.argmin(-1)
        return {
            "chosen": result.responses[rows, best], "chosen_mask": result.response_mask[rows, best].float(),
            "rejected": result.responses[rows, worst], "rejected_mask": result.response_mask[rows, worst].float(),
        }


@StrategyFactory.register("grpo")
class GRPOStrategy(BaseStrategy):
    """Group-relative PPO on response tokens with a k1-style KL penalty to a frozen reference model."""

    def __init__(self, model, device, old_model, ref_model, clip_eps: float = 0.2, kl_coef: float = 0.01,
                 group_size: int = 4, **kwargs):
        super().__init__(model, device, **kwargs)
        self.old_model, self.ref_model = old_model, ref_model
        self.clip_eps, self.kl_coef, self.group_size = clip_eps, kl_coef, group_size

    def sync_old_model(self):
        sd = self.executor.unwrap_model(self.model)
        if self.executor.use_distributed:
            sd = broadcast_state_dict(sd)
        if sd is not None:
            self.old_model.load_state_dict(sd)

    def compute_loss_output(self, batch) -> LossOutput:
        batch = self._to_rank(self._whole_sequences(batch))
        prompts, responses, masks, rewards = batch["prompts"], batch["responses"], batch["masks"], batch["rewards"]
        b, g, rlen = responses.shape
        resp = responses.reshape(b * g, rlen)
        rmask = masks.reshape(b * g, rlen)
        prompt = prompts[:, None].expand(-1, g, -1).reshape(b * g, -1)
        pmask = batch.get("prompt_mask")
        pmask = prompts.ne(0) if pmask is None else pmask
        pmask = pmask[:, None].expand(-1, g, -1).reshape(b * g, -1)
        plen = prompt.shape[1]
        seq = torch.cat([prompt, resp], dim=-1)
        loss_mask = torch.cat([torch.zeros_like(prompt, dtype=torch.bool), rmask.bool()], dim=-1)
        attn = padded_causal_attention(torch.cat([pmask.bool(), rmask.bool()], dim=-1))
        if isinstance(attn, Tensor):
            attn = attn.to(seq.device)

        def response_logprobs(model):
            out = get_logprobs(model, seq, attn, loss_mask, "none")
            return out["logprobs"][:, plen - 1:].reshape(b, g, -1), out

        lp_pol, pol = response_logprobs(self.model)
        with torch.no_grad():
            lp_old, _ = response_logprobs(self.old_model)
            lp_ref, _ = response_logprobs(self.ref_model)
        tok = rmask.reshape(b, g, -1).float()
        count = tok.sum().clamp(min=1.0)
        surrogate_sum, kl_sum = grpo_terms(lp_pol, lp_old, lp_ref, rewards, tok, self.clip_eps)
        policy_loss = surrogate_sum / count
        kl = self.kl_coef * kl_sum / count
        return self._loss_output(policy_loss + kl, {"policy_loss": policy_loss, "kl_loss": kl},
                                 pol["aux_loss"], pol.get("router_stats"))

    def supports_online(self) -> bool:
        return True

    def prepare_from_rollout(self, result: "RolloutResult") -> Dict[str, Tensor]:
        return {"prompts": result.prompts, "prompt_mask": result.prompt_mask, "responses": result.responses,
                "masks": result.response_mask, "rewards": result.rewards}

    def _on_rollout_refresh(self):
        self.sync_old_model()


StrategyFactory.register("online_grpo")(GRPOStrategy)
StrategyFactory.register("online_dpo")(DPOStrategy)
