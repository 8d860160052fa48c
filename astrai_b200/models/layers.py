"""Leaf modules: Linear, RMSNorm, Embedding, RotaryEmbedding.

Parameter names, shapes and initialisation follow the reference so that its checkpoints load unchanged
(``astrai/model/components/linear.py:7-24``, ``norm.py:7-15``, ``embedding.py:9-26``, ``rope.py:8-76``); the
math runs through :mod:`astrai_b200.ops`.
"""

from __future__ import annotations

import math
from typing import Dict, Optional

import torch
import torch.nn as nn
from torch import Tensor

from astrai_b200 import ops


class Linear(nn.Module):
    def __init__(self, in_dim: int, out_dim: int, bias: bool = False, init_std: float = 0.02):
        super().__init__()
        self.in_dim, self.out_dim, self.init_std = in_dim, out_dim, init_std
        self.weight = nn.Parameter(torch.empty(out_dim, in_dim))
        self.bias = nn.Parameter(torch.zeros(out_dim)) if bias else None

    def reset_parameters(self):
        nn.init.normal_(self.weight, mean=0.0, std=self.init_std)
        if self.bias is not None:
            bound = 1.0 / math.sqrt(self.in_dim)
            nn.init.uniform_(self.bias, -bound, bound)

    def forward(self, x: Tensor) -> Tensor:
        return ops.linear(x, self.weight, self.bias)

    def extra_repr(self):
        return f"in={self.in_dim}, out={self.out_dim}, bias={self.bias is not None}"


class RMSNorm(nn.Module):
    def __init__(self, dim: int, norm_eps: float):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.norm_eps = norm_eps

    def forward(self, x: Tensor, residual: Optional[Tensor] = None):
        """``rms_norm(x)``; with ``residual`` the pair ``(x + residual, rms_norm(x + residual))`` from one kernel."""
        if residual is not None:
            return ops.add_rms_norm(x, residual, self.weight, self.norm_eps)
        return ops.rms_norm(x, self.weight, self.norm_eps)


class Embedding(nn.Module):
    def __init__(self, vocab_size: int, embedding_dim: int, neftune_alpha: float = 0.0):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(vocab_size, embedding_dim))
        self.neftune_noise_alpha = neftune_alpha

    def set_neftune_alpha(self, alpha: float):
        self.neftune_noise_alpha = alpha

    def reset_parameters(self):
        nn.init.normal_(self.weight, mean=0.0, std=0.02)

    def forward(self, ids: Tensor) -> Tensor:
        out = ops.embedding(ids, self.weight)
        if self.training and self.neftune_noise_alpha > 0.0:
            # NEFTune: uniform-in-spirit noise scaled by alpha / sqrt(seq_len) (reference embedding.py:22-25 uses randn)
            out = out + (self.neftune_noise_alpha / math.sqrt(out.size(1))) * torch.randn_like(out)
        return out


def rope_table(dim: int, max_len: int, base: float = 10000.0, device=None) -> Tensor:
    """``[max_len, dim/2, 2]`` fp32 (cos, sin), angles computed in fp64."""
    inv = base ** (-torch.arange(0, dim, 2, dtype=torch.float64, device=device) / dim)
    ang = torch.outer(torch.arange(max_len, dtype=torch.float64, device=device), inv).float()
    return torch.stack((ang.cos(), ang.sin()), dim=-1)


def ntk_base(base: float, dim: int, factor: float) -> float:
    """NTK-aware rescaling of the rotary base for a context ``factor`` times longer (``astrai/model/components/rope.py:27-28``)."""
    return base * factor ** (dim / (dim - 2))


def get_rotary_emb(dim: int, max_len: int, base: float = 10000.0, device=None) -> Tensor:
    """The (cos, sin) table ``[max_len, dim / 2, 2]`` under the reference's name (``astrai/model/components/rope.py:8-24``)."""
    return rope_table(dim, max_len, base, device)


def apply_rotary_emb(x: Tensor, freqs_cis: Tensor) -> Tensor:
    """Rotate ``x [..., heads, head_dim]`` by ``freqs_cis [..., head_dim / 2, 2]`` (adjacent pairs, fp32 math)."""
    return ops.rotary(x, freqs_cis)


class RotaryEmbedding(nn.Module):
    """Position -> (cos, sin) rows.  ``rope_scaling={"type": "ntk", "factor": f}`` rescales the base by
    ``f ** (dim / (dim - 2))``; other types are accepted and leave the base alone, as in the reference."""

    def __init__(self, dim: int, max_len: int, base: float = 10000.0, rope_scaling: Optional[Dict] = None):
        super().__init__()
        self.dim, self.max_len, self.rope_scaling = dim, max_len, rope_scaling
        if rope_scaling is not None and rope_scaling.get("type", "ntk") == "ntk":
            base = ntk_base(base, dim, rope_scaling.get("factor", 1.0))
        self.base = base
        self.register_buffer("freqs_cis", rope_table(dim, max_len, base), persistent=False)

    def _apply(self, fn, *a, **kw):
        # The table stays fp32 whatever dtype the model is cast to: rebuild it on the new device if a cast hit it.
        out = super()._apply(fn, *a, **kw)
        if self.freqs_cis.dtype != torch.float32:
            self.freqs_cis = rope_table(self.dim, self.max_len, self.base, device=self.freqs_cis.device)
        return out

    def forward(self, x: Tensor, position_ids: Optional[Tensor] = None) -> Tensor:
        if position_ids is None:
            if x.ndim == 2:  # packed [tokens, dim]
                position_ids = torch.arange(x.size(0), device=x.device)
            else:
                position_ids = torch.arange(x.size(1), device=x.device).expand(x.size(0), -1)
        return self.freqs_cis[position_ids]
