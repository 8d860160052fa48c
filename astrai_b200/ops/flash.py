"""Differentiable front end of the tcgen05 flash-attention kernels (``flash_fwd.cu`` / ``flash_bwd.cu``).

Tensors are packed along tokens: ``q [Tq, Hq, D]``, ``k / v [Tk, Hkv, D]``; a dense ``[B, S, H, D]`` batch is the same
memory viewed as ``[B*S, H, D]`` with a fixed sequence length.  Variable-length batches (packed documents, ragged
prefill) pass ``cu_seqlens`` (int32 ``[B+1]``).  Causal masking is lower-right aligned, so the same call serves
training (``k_len == q_len``) and prefill on top of cached keys (``k_len > q_len``).

Plays the role of ``F.scaled_dot_product_attention`` / ``flash_attn_varlen_func`` in the reference
(``astrai/extension/backend/attention.py:453-468``, ``:663-702``).
"""

from __future__ import annotations

from typing import Optional

import torch
from torch import Tensor
from torch.autograd import Function

from astrai_b200.ops import native

SUPPORTED_HEAD_DIMS = (64, 128)


def _packed_ok(t: Tensor) -> bool:
    return (t.dim() == 3 and t.dtype == torch.bfloat16 and t.stride(2) == 1 and t.stride(1) == t.shape[2]
            and t.stride(0) % 8 == 0 and t.data_ptr() % 16 == 0)


def _fix(t: Tensor) -> Tensor:
    return t if _packed_ok(t) else t.contiguous()


class _FlashFn(Function):
    @staticmethod
    def forward(ctx, q, k, v, cu_q, cu_k, batch, sq, sk, max_q, max_k, causal, scale):
        q, k, v = _fix(q), _fix(k), _fix(v)
        out, lse = torch.ops.astrai_b200.flash_fwd(q, k, v, cu_q, cu_k, batch, sq, sk, max_q, causal, scale)
        ctx.save_for_backward(q, k, v, out, lse, *([cu_q, cu_k] if cu_q is not None else []))
        ctx.meta = (batch, sq, sk, max_q, max_k, causal, scale, cu_q is not None)
        return out

    @staticmethod
    def backward(ctx, dout):
        batch, sq, sk, max_q, max_k, causal, scale, varlen = ctx.meta
        saved = ctx.saved_tensors
        q, k, v, out, lse = saved[:5]
        cu_q, cu_k = (saved[5], saved[6]) if varlen else (None, None)
        dq, dk, dv = torch.ops.astrai_b200.flash_bwd(q, k, v, out, _fix(dout), lse, cu_q, cu_k, batch, sq, sk, max_q, max_k,
                                                     causal, scale)
        return dq, dk, dv, None, None, None, None, None, None, None, None, None


def supported(q: Tensor, k: Tensor, v: Tensor) -> bool:
    return (q.is_cuda and q.dtype == torch.bfloat16 and k.dtype == torch.bfloat16 and v.dtype == torch.bfloat16
            and q.shape[-1] in SUPPORTED_HEAD_DIMS and q.shape[-1] == k.shape[-1] == v.shape[-1]
            and q.shape[-2] % k.shape[-2] == 0)


def flash_attention(q: Tensor, k: Tensor, v: Tensor, causal: bool = True, scale: Optional[float] = None) -> Tensor:
    """Dense batch: ``q [B, Sq, Hq, D]``, ``k / v [B, Sk, Hkv, D]`` -> ``[B, Sq, Hq, D]``."""
    native.require()
    b, sq, hq, d = q.shape
    sk, hkv = k.shape[1], k.shape[2]
    scale = float(scale) if scale is not None else d ** -0.5
    out = _FlashFn.apply(q.reshape(b * sq, hq, d), k.reshape(b * sk, hkv, d), v.reshape(b * sk, hkv, d), None, None,
                         b, sq, sk, sq, sk, bool(causal), scale)
    return out.view(b, sq, hq, d)


def flash_attention_varlen(q: Tensor, k: Tensor, v: Tensor, cu_seqlens_q: Tensor, cu_seqlens_k: Tensor, max_q: int,
                           max_k: int, causal: bool = True, scale: Optional[float] = None) -> Tensor:
    """Packed batch: ``q [Tq, Hq, D]``, ``k / v [Tk, Hkv, D]`` with int32 ``cu_seqlens`` ``[B+1]`` on the device."""
    native.require()
    d = q.shape[-1]
    scale = float(scale) if scale is not None else d ** -0.5
    batch = cu_seqlens_q.numel() - 1
    return _FlashFn.apply(q, k, v, cu_seqlens_q.int(), cu_seqlens_k.int(), batch, 0, 0, int(max_q), int(max_k),
                          bool(causal), scale)


PAGED_PAGE_SIZES = (8, 16, 32, 64)


@torch.no_grad()
def flash_attention_paged(q: Tensor, k_pool: Tensor, v_pool: Tensor, cu_seqlens_q: Tensor, cu_seqlens_k: Tensor,
                          req_to_token: Tensor, req_pool_indices: Tensor, page_size: int, max_q: int, causal: bool = True,
                          scale: Optional[float] = None) -> Tensor:
    """Ragged prefill straight over the paged KV pool (inference, forward only): the kernel's TMA producer walks the
    slot table page by page, so the batch's keys are never gathered into a packed copy first.

    ``q [Tq, Hq, D]`` packed queries; ``k_pool / v_pool [n_slots, Hkv, D]``; ``cu_seqlens_k`` carries the key counts
    (cached prefix + new tokens); request ``b`` finds the slot of its key ``t`` at ``req_to_token[req_pool_indices[b], t]``
    and the ``page_size`` tokens of a page occupy consecutive, page-aligned slots.  Causal masking is lower-right
    aligned.  The reference's paged-prefill kernel addresses K / V the same way
    (``csrc/kernels/attention/layout_policies.cuh:39-255``)."""
    native.require()
    scale = float(scale) if scale is not None else q.shape[-1] ** -0.5
    return torch.ops.astrai_b200.flash_fwd_paged(_fix(q), k_pool, v_pool, cu_seqlens_q.int(), cu_seqlens_k.int(), req_to_token,
                                                 req_pool_indices.int(), int(page_size), int(max_q), bool(causal), scale)
