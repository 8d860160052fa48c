"""Plain-PyTorch statements of every op: the CPU path and the oracle the CUDA kernels are tested against."""

from __future__ import annotations

import torch
import torch.nn.functional as F
from torch import Tensor


def rms_norm(x: Tensor, weight: Tensor, eps: float) -> Tensor:
    return F.rms_norm(x, (x.shape[-1],), weight, eps)


def rotary(x: Tensor, freqs: Tensor) -> Tensor:
    """Interleaved-pair rotation.  x [..., H, D]; freqs [..., D/2, 2] holding (cos, sin)."""
    cos = freqs[..., 0].unsqueeze(-2)
    sin = freqs[..., 1].unsqueeze(-2)
    xf = x.float().unflatten(-1, (-1, 2))
    x0, x1 = xf[..., 0], xf[..., 1]
    out = torch.stack((x0 * cos - x1 * sin, x0 * sin + x1 * cos), dim=-1).flatten(-2)
    return out.to(x.dtype)


def swiglu(gate: Tensor, up: Tensor) -> Tensor:
    return up * F.silu(gate)


def linear(x: Tensor, weight: Tensor, bias=None) -> Tensor:
    return F.linear(x, weight, bias)


def cross_entropy_rows(logits: Tensor, targets: Tensor, label_smoothing: float = 0.0, ignore_index: int = -100) -> Tensor:
    """Per-row loss in fp32 (0 where the target is ignored)."""
    return F.cross_entropy(
        logits.float(), targets, reduction="none", label_smoothing=label_smoothing, ignore_index=ignore_index
    )


def token_logprobs(logits: Tensor, ids: Tensor) -> Tensor:
    return torch.log_softmax(logits.float(), dim=-1).gather(-1, ids.unsqueeze(-1)).squeeze(-1)


def attention(q: Tensor, k: Tensor, v: Tensor, mask=None, causal: bool = False, scale=None) -> Tensor:
    """q [B,S,Hq,D], k/v [B,L,Hkv,D] -> [B,S,Hq,Dv]; bool mask broadcastable to [B,Hq,S,L] (True = attend)."""
    hq, hkv = q.shape[2], k.shape[2]
    qt, kt, vt = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
    if hq != hkv:
        kt = kt.repeat_interleave(hq // hkv, dim=1)
        vt = vt.repeat_interleave(hq // hkv, dim=1)
    out = F.scaled_dot_product_attention(qt, kt, vt, attn_mask=mask, is_causal=causal and mask is None, scale=scale)
    return out.transpose(1, 2)
