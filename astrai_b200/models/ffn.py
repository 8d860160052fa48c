"""Feed-forward blocks: SwiGLU MLP and DeepSeek-style mixture of experts.

Semantics follow ``astrai/model/components/mlp.py:32-172``: ``down(up(x) * silu(gate(x)))``; MoE = mean of the
shared experts + sum over the top-k routed experts weighted by (optionally renormalised) softmax probabilities;
auxiliary loss ``E * sum_e(load_e * mean_prob_e)`` while training.  Unlike the reference's per-expert Python loop
with a host sync per layer, routed tokens are processed from one expert-sorted buffer; the per-expert segment
sizes stay on the device when the grouped kernel is available.
"""

from __future__ import annotations

from typing import Optional, TypedDict

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch import Tensor

from astrai_b200 import ops
from astrai_b200.factory import BaseFactory
from astrai_b200.models.layers import Linear


class FFNFactory(BaseFactory[nn.Module]):
    pass


class RouterStats(TypedDict):
    probs: Tensor
    topk_indices: Tensor


class FFNOutput(TypedDict):
    hidden_states: Tensor
    aux_loss: Optional[Tensor]
    router_stats: Optional[RouterStats]


@FFNFactory.register("mlp")
class MLP(nn.Module):
    def __init__(self, dim: int, dim_ffn: int, down_init_std: float = 0.02):
        super().__init__()
        self.up = Linear(dim, dim_ffn)
        self.gate = Linear(dim, dim_ffn)
        self.down = Linear(dim_ffn, dim, init_std=down_init_std)
        self.fused_gate_up = None  # set by flat-buffer executors: view [2*dim_ffn, dim] = gate rows then up rows

    def hidden(self, x: Tensor) -> Tensor:
        w = self.fused_gate_up
        if w is not None and x.is_cuda:
            return ops.swiglu_fused(ops.linear(x, w, None, grad_owner=w))
        return ops.swiglu(self.gate(x), self.up(x))

    def forward(self, x: Tensor) -> FFNOutput:
        return {"hidden_states": self.down(self.hidden(x)), "aux_loss": None, "router_stats": None}


@FFNFactory.register("moe")
class DeepSeekMoE(nn.Module):
    def __init__(self, dim: int, dim_ffn: int, n_routed_experts: int, n_shared_experts: int = 1,
                 n_activated_experts: int = 2, topk_method: str = "greedy", n_layers: int = 1,
                 moe_intermediate_size: Optional[int] = None, shared_expert_intermediate_size: Optional[int] = None,
                 norm_topk_prob: bool = True):
        super().__init__()
        if not n_routed_experts or not n_activated_experts:
            raise ValueError("a mixture-of-experts layer needs n_routed_experts and n_activated_experts "
                             f"(got {n_routed_experts!r} and {n_activated_experts!r})")
        self.dim = dim
        self.n_routed_experts = n_routed_experts
        self.n_shared_experts = n_shared_experts or 0
        self.n_activated_experts = n_activated_experts
        self.topk_method = topk_method  # stored for config round trips; routing is softmax -> top-k
        self.norm_topk_prob = norm_topk_prob
        expert_ffn = moe_intermediate_size if moe_intermediate_size is not None else dim_ffn
        shared_ffn = shared_expert_intermediate_size if shared_expert_intermediate_size is not None else dim_ffn
        self.router = Linear(dim, n_routed_experts)
        moe_scale = 1 / max(self.n_shared_experts, 1) + 1 / n_activated_experts
        std = 0.02 / (2 * n_layers * moe_scale) ** 0.5
        self.shared_experts = nn.ModuleList(MLP(dim, shared_ffn, std) for _ in range(self.n_shared_experts))
        self.routed_experts = nn.ModuleList(MLP(dim, expert_ffn, std) for _ in range(n_routed_experts))
        self.expert_parallel = False  # set by the expert-parallel executor once `routed_experts` is its stacked, sharded form
        self.stacked_experts = None  # set for serving: ([E, 2F, D] gate|up, [E, D, F] down) that the experts' weights view

    # ---- routing --------------------------------------------------------------------------------------------
    def _use_kernels(self, x: Tensor) -> bool:
        from astrai_b200.ops import moe

        ffn = self.routed_experts[0].gate.weight.shape[0]
        return (not self.expert_parallel and moe.available(x, self.n_routed_experts, self.n_activated_experts)
                and ffn % 64 == 0 and all(type(m.gate).__name__ == "Linear" for m in self.routed_experts))

    def _forward_kernels(self, x: Tensor, with_aux: bool):
        """Router, dispatch, two grouped GEMMs with SwiGLU in between, and combine on the sm_100a kernels."""
        from astrai_b200.ops import moe

        e, k = self.n_routed_experts, self.n_activated_experts
        logits = self.router(x)
        probs, idx, weights, counts, psum = moe.route(logits, k, self.norm_topk_prob)
        aux, stats = None, None
        if with_aux:
            load = counts.float() / idx.numel()
            aux = e * (load * (psum / x.shape[0])).sum()
            stats = {"probs": probs.detach(), "topk_indices": idx}
        xs, plan = moe.dispatch(x, idx, counts, e)
        if self.stacked_experts is not None and not torch.is_grad_enabled():
            w_gu, w_dn = self.stacked_experts  # serving: the experts' parameters are views of these two tensors
        else:
            w_gu = torch.stack([torch.cat([m.gate.weight, m.up.weight], dim=0) for m in self.routed_experts])  # [E, 2F, D]
            w_dn = torch.stack([m.down.weight for m in self.routed_experts])                                   # [E, D, F]
        h = ops.swiglu_fused(moe.zero_unused_rows(moe.grouped_linear(xs, w_gu, plan), plan))
        y = moe.zero_unused_rows(moe.grouped_linear(h, w_dn, plan), plan)
        return moe.combine(y, weights, plan), aux, stats

    def route(self, x: Tensor, with_aux: bool):
        e, k = self.n_routed_experts, self.n_activated_experts
        probs = torch.softmax(self.router(x).float(), dim=-1).to(x.dtype)
        weights, idx = torch.topk(probs, k, dim=-1, sorted=False)
        if self.norm_topk_prob:
            weights = weights / weights.sum(dim=-1, keepdim=True)
        aux, stats = None, None
        if with_aux:
            load = torch.zeros(e, dtype=torch.float32, device=x.device)
            load.scatter_add_(0, idx.reshape(-1), torch.ones(idx.numel(), dtype=torch.float32, device=x.device))
            load = load / idx.numel()
            aux = e * (load * probs.float().mean(dim=0)).sum()
            stats = {"probs": probs.detach(), "topk_indices": idx}
        return weights, idx, aux, stats

    # ---- expert compute ---------------------------------------------------------------------------------------
    def _experts_sorted(self, tokens: Tensor, counts: Tensor) -> Tensor:
        """Run every expert on its contiguous slice of the expert-sorted token buffer."""
        out = torch.empty_like(tokens)
        bounds = torch.cumsum(counts, 0).tolist()
        start = 0
        for eid, end in enumerate(bounds):
            if end > start:
                out[start:end] = self.routed_experts[eid](tokens[start:end])["hidden_states"]
            start = end
        return out

    def _routed(self, x: Tensor, weights: Tensor, idx: Tensor) -> Tensor:
        n, _ = x.shape
        k, e = self.n_activated_experts, self.n_routed_experts
        flat = idx.reshape(-1)
        order = torch.argsort(flat, stable=True)
        counts = torch.bincount(flat, minlength=e)
        src_tok = order // k
        y = self._experts_sorted(x[src_tok], counts)
        y = y * weights.reshape(-1, 1)[order]
        out = torch.zeros_like(x)
        out.index_add_(0, src_tok, y)
        return out

    def _forward_expert_parallel(self, x: Tensor, with_aux: bool):
        """Local routing, then the routed experts of every rank of the expert-parallel group (tokens travel to the
        experts' owners and back inside ``self.routed_experts``).  The auxiliary loss uses this rank's tokens."""
        from astrai_b200.ops import moe

        e, k = self.n_routed_experts, self.n_activated_experts
        if moe.available(x, e, k):
            probs, idx, weights, counts, psum = moe.route(self.router(x), k, self.norm_topk_prob)
            aux = stats = None
            if with_aux:
                aux = e * ((counts.float() / idx.numel()) * (psum / x.shape[0])).sum()
                stats = {"probs": probs.detach(), "topk_indices": idx}
        else:
            weights, idx, aux, stats = self.route(x, with_aux)
            counts = torch.bincount(idx.reshape(-1), minlength=e).to(torch.int32)
        return self.routed_experts(x, idx, weights, counts), aux, stats

    def forward(self, x: Tensor) -> FFNOutput:
        with_aux = self.training and torch.is_grad_enabled()
        shape = x.shape
        flat = x.reshape(-1, shape[-1])
        if self.expert_parallel:
            out, aux, stats = self._forward_expert_parallel(flat, with_aux)
        elif self._use_kernels(flat):
            out, aux, stats = self._forward_kernels(flat, with_aux)
        else:
            weights, idx, aux, stats = self.route(flat, with_aux)
            out = self._routed(flat, weights, idx)
        if self.n_shared_experts:
            shared = self.shared_experts[0](flat)["hidden_states"]
            for ex in self.shared_experts[1:]:
                shared = shared + ex(flat)["hidden_states"]
            out = out + shared / self.n_shared_experts
        return {"hidden_states": out.view(shape), "aux_loss": aux, "router_stats": stats}
