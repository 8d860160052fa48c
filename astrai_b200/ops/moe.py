"""Differentiable mixture-of-experts primitives on the sm_100a kernels (``moe.cu``, ``gemm_grouped.cu``).

``route`` -> ``dispatch`` -> ``grouped_linear`` (x2 with SwiGLU in between) -> ``combine``: token rows are moved once
into expert-sorted segments padded to 128 rows, the expert matrices run as grouped tcgen05 GEMMs driven by a device-side
tile -> expert table, and the weighted sum over each token's choices is a gather.  Nothing is read back to the host.
Semantics follow ``astrai/model/components/mlp.py:95-172`` of the reference.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch
from torch import Tensor
from torch.autograd import Function

from astrai_b200.ops import native

TILE = 128


def available(x: Tensor, n_experts: int, k: int) -> bool:
    return (x.is_cuda and x.dtype == torch.bfloat16 and n_experts <= 256 and k <= 8 and x.shape[-1] % 64 == 0
            and native.is_available())


class _RouteFn(Function):
    """probs = softmax(logits) (rounded to the activation dtype), top-k, optional renormalisation."""

    @staticmethod
    def forward(ctx, logits: Tensor, k: int, renorm: bool):
        probs, idx, w, counts, psum = torch.ops.astrai_b200.moe_router(logits.contiguous(), k, renorm)
        ctx.save_for_backward(probs, idx, w)
        ctx.renorm = renorm
        ctx.mark_non_differentiable(idx, counts)
        return probs, idx, w, counts, psum

    @staticmethod
    def backward(ctx, dprobs, _didx, dw, _dcounts, dpsum):
        probs, idx, w = ctx.saved_tensors
        p = probs.float()
        g = torch.zeros_like(p) if dprobs is None else dprobs.float().clone()
        if dpsum is not None:
            g += dpsum.float()[None, :]
        if dw is not None:
            dwf = dw.float()
            if ctx.renorm:  # w = p_k / s, s = sum of the selected p
                sel = p.gather(1, idx)
                s = sel.sum(1, keepdim=True)
                dsel = dwf / s - (dwf * sel).sum(1, keepdim=True) / (s * s)
            else:
                dsel = dwf
            g.scatter_add_(1, idx, dsel)
        dlogits = p * (g - (g * p).sum(1, keepdim=True))
        return dlogits.to(probs.dtype), None, None


def route(logits: Tensor, k: int, renorm: bool):
    """``(probs [T,E], idx [T,K] int64, weights [T,K], counts [E] int32, prob_sums [E] fp32)``."""
    native.require()
    return _RouteFn.apply(logits, k, renorm)


@dataclass
class Plan:
    offsets: Tensor      # [E+1] padded segment starts
    tile_expert: Tensor  # [max_tiles] expert of every 128-row tile, -1 when unused
    slot_of: Tensor      # [T, K] row of every (token, choice) in the sorted buffer
    max_rows: int


class _DispatchFn(Function):
    @staticmethod
    def forward(ctx, x: Tensor, idx: Tensor, counts: Tensor, n_experts: int):
        t, k = idx.shape
        max_rows = -(-(t * k) // TILE) * TILE + n_experts * TILE
        offsets, tile_expert, cursors, _total = torch.ops.astrai_b200.moe_plan(counts, max_rows // TILE)
        sorted_x, slot_of = torch.ops.astrai_b200.moe_permute(x.contiguous(), idx.contiguous(), counts, offsets, cursors, max_rows)
        ctx.save_for_backward(slot_of)
        ctx.mark_non_differentiable(offsets, tile_expert, slot_of)
        return sorted_x, offsets, tile_expert, slot_of

    @staticmethod
    def backward(ctx, dsorted, *_):
        (slot_of,) = ctx.saved_tensors
        return torch.ops.astrai_b200.moe_combine(dsorted.contiguous(), slot_of, None), None, None, None


def dispatch(x: Tensor, idx: Tensor, counts: Tensor, n_experts: int) -> Tuple[Tensor, Plan]:
    sorted_x, offsets, tile_expert, slot_of = _DispatchFn.apply(x, idx, counts, n_experts)
    return sorted_x, Plan(offsets, tile_expert, slot_of, sorted_x.shape[0])


class _GroupedLinearFn(Function):
    @staticmethod
    def forward(ctx, x: Tensor, w: Tensor, tile_expert: Tensor, offsets: Tensor):
        ctx.save_for_backward(x, w, tile_expert, offsets)
        return torch.ops.astrai_b200.grouped_gemm_rows(x, w.contiguous(), True, tile_expert)

    @staticmethod
    def backward(ctx, dy: Tensor):
        x, w, tile_expert, offsets = ctx.saved_tensors
        dy = dy.contiguous()
        dx = torch.ops.astrai_b200.grouped_gemm_rows(dy, w.contiguous(), False, tile_expert) if ctx.needs_input_grad[0] else None
        dw = torch.ops.astrai_b200.grouped_gemm_wgrad(dy, x, offsets, False) if ctx.needs_input_grad[1] else None
        return dx, dw, None, None


def grouped_linear(x_sorted: Tensor, w_stacked: Tensor, plan: Plan) -> Tensor:
    """``y[r] = x[r] @ w[e(r)].T`` for expert-sorted rows; ``w_stacked`` is ``[E, N, K]``.

    Rows of unused tiles are left uninitialised; rows of padding are zero when the input padding is zero."""
    return _GroupedLinearFn.apply(x_sorted, w_stacked, plan.tile_expert, plan.offsets)


class _CombineFn(Function):
    @staticmethod
    def forward(ctx, y: Tensor, weights: Tensor, slot_of: Tensor):
        ctx.save_for_backward(y, weights, slot_of)
        return torch.ops.astrai_b200.moe_combine(y.contiguous(), slot_of, weights.contiguous())

    @staticmethod
    def backward(ctx, dout: Tensor):
        y, weights, slot_of = ctx.saved_tensors
        dy, dw = torch.ops.astrai_b200.moe_combine_bwd(dout.contiguous(), y.contiguous(), slot_of, weights.contiguous())
        return dy, dw.to(weights.dtype), None


def combine(y_sorted: Tensor, weights: Tensor, plan: Plan) -> Tensor:
    """``out[t] = sum_k weights[t,k] * y_sorted[slot[t,k]]``."""
    return _CombineFn.apply(y_sorted, weights, plan.slot_of)


def zero_unused_rows(t: Tensor, plan: Plan) -> Tensor:
    """Rows past the last segment were never written by the grouped GEMM: blank them before they are consumed again."""
    used = plan.offsets[-1]
    rows = torch.arange(t.shape[0], device=t.device)
    return torch.where((rows < used)[:, None], t, torch.zeros((), dtype=t.dtype, device=t.device))
