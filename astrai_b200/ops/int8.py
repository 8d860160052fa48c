"""W8A8 int8 linear layers on the ``tcgen05.mma kind::i8`` GEMM (``ops/csrc/gemm_fp8.cu``).

Activations are quantised per token (one fp32 scale per row, computed on the fly), weights per output channel (one scale
per row of the ``[out, in]`` matrix, computed once).  The integer product is exact (int32 accumulation in tensor
memory); the epilogue multiplies by ``row_scale[m] * col_scale[n]`` and adds the bias.  Meant for inference: there is no
backward pass.  The reference has no int8 path; its quantised path is per-tensor fp8 only
(``astrai/extension/fp8.py:108-187``).
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch
from torch import Tensor, nn

from astrai_b200.ops import native


def eligible(x: Tensor, in_features: int) -> bool:
    return x.is_cuda and x.dtype == torch.bfloat16 and in_features % 16 == 0 and native.is_available()


def quantize_rows(x: Tensor) -> Tuple[Tensor, Tensor]:
    """``(q int8 [R, C], scale fp32 [R])`` with ``scale = max|x[r]| / 127`` and ``q = round(x / scale)``."""
    if x.is_cuda:
        native.require()
        return torch.ops.astrai_b200.int8_quantize_rows(x.contiguous())
    return quantize_rows_reference(x)


def quantize_rows_reference(x: Tensor) -> Tuple[Tensor, Tensor]:
    """Plain PyTorch statement of :func:`quantize_rows` (CPU path, tests)."""
    xf = x.float()
    amax = xf.abs().amax(dim=1)
    scale = torch.where(amax > 0, amax / 127.0, torch.ones_like(amax))
    q = torch.clamp(torch.round(xf / scale[:, None]), -127, 127).to(torch.int8)
    return q, scale


def mm_int8(a_q: Tensor, a_scale: Tensor, b_q: Tensor, b_scale: Tensor, bias: Optional[Tensor] = None) -> Tensor:
    """``(a_q @ b_q.T) * a_scale[:, None] * b_scale[None, :] (+ bias)`` as bf16; ``a_q`` ``[M, K]``, ``b_q`` ``[N, K]`` int8."""
    if a_q.is_cuda:
        native.require()
        return torch.ops.astrai_b200.int8_gemm(a_q.contiguous(), b_q.contiguous(), a_scale.contiguous(), b_scale.contiguous(),
                                               None if bias is None else bias.to(torch.bfloat16).contiguous())
    out = (a_q.float() @ b_q.float().t()) * a_scale[:, None] * b_scale[None, :]
    if bias is not None:
        out = out + bias.float()
    return out.to(torch.bfloat16)


def int8_linear(x: Tensor, w_q: Tensor, w_scale: Tensor, bias: Optional[Tensor] = None) -> Tensor:
    """``x @ W.T`` with the activations quantised per token on the fly; ``x`` ``[..., in]`` bf16."""
    shape = x.shape
    a_q, a_scale = quantize_rows(x.reshape(-1, shape[-1]))
    return mm_int8(a_q, a_scale, w_q, w_scale, bias).view(*shape[:-1], w_q.shape[0])


class Int8Linear(nn.Module):
    """Inference-only replacement of a linear layer: int8 weight + per-channel scale (buffers, saved with the model)."""

    def __init__(self, in_features: int, out_features: int, bias: bool = False, device=None):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.register_buffer("weight_q", torch.zeros(out_features, in_features, dtype=torch.int8, device=device))
        self.register_buffer("weight_scale", torch.ones(out_features, dtype=torch.float32, device=device))
        self.register_buffer("bias", torch.zeros(out_features, dtype=torch.bfloat16, device=device) if bias else None)

    @classmethod
    def from_linear(cls, linear: nn.Module) -> "Int8Linear":
        w = linear.weight.detach()
        b = getattr(linear, "bias", None)
        out = cls(w.shape[1], w.shape[0], bias=b is not None, device=w.device)
        q, s = quantize_rows(w.to(torch.bfloat16))
        out.weight_q.copy_(q)
        out.weight_scale.copy_(s)
        if b is not None:
            out.bias.copy_(b.detach().to(torch.bfloat16))
        return out

    def forward(self, x: Tensor) -> Tensor:
        return int8_linear(x.to(torch.bfloat16), self.weight_q, self.weight_scale, self.bias)


def quantize_model_int8(model: nn.Module, skip=("lm_head", "router")) -> int:
    """Swap every linear layer (an ``nn.Module`` with a 2-D ``weight`` whose input size is a multiple of 16) except the
    named ones for :class:`Int8Linear`; returns how many were replaced.  For serving: call after loading the weights."""
    replaced = 0
    for name, parent in list(model.named_modules()):
        for child_name, child in list(parent.named_children()):
            w = getattr(child, "weight", None)
            is_linear = (isinstance(child, nn.Linear) or type(child).__name__ == "Linear") and w is not None and w.dim() == 2
            if not is_linear or any(s in child_name for s in skip) or w.shape[1] % 16:
                continue
            setattr(parent, child_name, Int8Linear.from_linear(child))
            replaced += 1
    return replaced
