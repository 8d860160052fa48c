"""Attention blocks: grouped-query attention and multi-head latent attention.

Op order (reference ``astrai/model/components/attention.py:69-85``, ``:146-181``): projections -> RoPE on q, k
-> optional per-head RMSNorm -> attention -> optional sigmoid gate -> output projection.  Sub-module names are
the checkpoint keys (``q_proj``, ``k_proj``, ``v_proj``, ``o_proj``, ``q_norm``, ``k_norm``, ``gate``,
``kv_a_proj``, ``kv_norm``, ``kv_b_proj``).

``GQA`` runs q/k/v as ONE tcgen05 GEMM when an executor has laid the three weights out back to back in a flat
buffer (it then sets ``fused_qkv`` to a view over them); RoPE and the head split are one kernel after it.
MLA additionally supports ``q_lora_rank`` (low-rank query, ``q_a_proj -> q_a_norm -> q_b_proj``), which the
reference lacks.
"""

from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn
from torch import Tensor

from astrai_b200 import ops
from astrai_b200.factory import BaseFactory
from astrai_b200.models.layers import Linear, RMSNorm
from astrai_b200.ops.attention import attention


class AttnFactory(BaseFactory[nn.Module]):
    pass


def _o_std(n_layers: int) -> float:
    return 0.02 / (2 * n_layers) ** 0.5


@AttnFactory.register("gqa")
class GQA(nn.Module):
    def __init__(self, dim: int, n_heads: int, n_kv_heads: int, use_qk_norm: bool, norm_eps: float,
                 use_gated_attention: bool, layer_id: int, n_layers: int = 1):
        super().__init__()
        if dim % n_heads or n_heads % n_kv_heads:
            raise ValueError("dim must divide by n_heads and n_heads by n_kv_heads")
        self.dim, self.n_heads, self.n_kv_heads, self.layer_id = dim, n_heads, n_kv_heads, layer_id
        self.head_dim = dim // n_heads
        self.n_rep = n_heads // n_kv_heads
        self.use_qk_norm, self.use_gated_attention = bool(use_qk_norm), bool(use_gated_attention)
        self.q_proj = Linear(dim, n_heads * self.head_dim)
        self.k_proj = Linear(dim, n_kv_heads * self.head_dim)
        self.v_proj = Linear(dim, n_kv_heads * self.head_dim)
        self.o_proj = Linear(dim, dim, init_std=_o_std(n_layers))
        if self.use_qk_norm:
            self.q_norm = RMSNorm(self.head_dim, norm_eps)
            self.k_norm = RMSNorm(self.head_dim, norm_eps)
        if self.use_gated_attention:
            self.gate = Linear(dim, dim)
        self.fused_qkv = None  # set by flat-buffer executors: tensor view [(Hq+2Hkv)*D, dim] with .main_grad

    def _project(self, x: Tensor, rotary_emb: Tensor):
        hq, hkv, d = self.n_heads, self.n_kv_heads, self.head_dim
        lead = x.shape[:-1]
        w = self.fused_qkv
        if w is not None and x.is_cuda:
            qkv = ops.linear(x.reshape(-1, self.dim), w, None, grad_owner=w)
            q, k, v = ops.qkv_rope(qkv, rotary_emb, hq, hkv, d)
            return q.view(*lead, hq, d), k.view(*lead, hkv, d), v.view(*lead, hkv, d)
        q = self.q_proj(x).view(*lead, hq, d)
        k = self.k_proj(x).view(*lead, hkv, d)
        v = self.v_proj(x).view(*lead, hkv, d)
        return ops.rotary(q, rotary_emb), ops.rotary(k, rotary_emb), v

    def forward(self, x: Tensor, rotary_emb: Tensor, attn_mask: Optional[Tensor] = None, kv_cache=None,
                is_causal: bool = False, fwd: Optional[str] = None) -> Tensor:
        q, k, v = self._project(x, rotary_emb)
        if self.use_qk_norm:
            q, k = self.q_norm(q), self.k_norm(k)
        out = attention(q, k, v, kv_cache, self.layer_id, attn_mask, is_causal, fwd).reshape(*x.shape[:-1], self.n_heads * self.head_dim)
        if self.use_gated_attention:
            out = out * torch.sigmoid(self.gate(x))
        return self.o_proj(out)


@AttnFactory.register("mla")
class MLA(nn.Module):
    def __init__(self, dim: int, n_heads: int, n_kv_heads: int, kv_lora_rank: int, qk_nope_head_dim: int,
                 qk_rope_head_dim: int, norm_eps: float, use_qk_norm: bool, use_gated_attention: bool, layer_id: int,
                 n_layers: int = 1, q_lora_rank: Optional[int] = None, v_head_dim: Optional[int] = None):
        super().__init__()
        self.dim, self.n_heads, self.n_kv_heads, self.layer_id = dim, n_heads, n_kv_heads, layer_id
        self.kv_lora_rank, self.q_lora_rank = kv_lora_rank, q_lora_rank
        self.qk_nope_head_dim, self.qk_rope_head_dim = qk_nope_head_dim, qk_rope_head_dim
        self.head_dim = qk_nope_head_dim + qk_rope_head_dim
        # value width per head: the reference ties it to the query / key width (and so needs heads * (nope + rope) == dim);
        # ``v_head_dim`` unties it (DeepSeek-style 192-wide scores with 128-wide values)
        self.v_head_dim = v_head_dim or self.head_dim
        self.n_rep = n_heads // n_kv_heads
        self.use_qk_norm, self.use_gated_attention = bool(use_qk_norm), bool(use_gated_attention)
        if q_lora_rank:
            self.q_a_proj = Linear(dim, q_lora_rank)
            self.q_a_norm = RMSNorm(q_lora_rank, norm_eps)
            self.q_b_proj = Linear(q_lora_rank, n_heads * self.head_dim)
        else:
            self.q_proj = Linear(dim, n_heads * self.head_dim)
        if self.use_qk_norm:
            self.q_norm = RMSNorm(self.head_dim, norm_eps)
            self.k_norm = RMSNorm(self.head_dim, norm_eps)
        self.kv_a_proj = Linear(dim, kv_lora_rank)
        self.kv_norm = RMSNorm(kv_lora_rank, norm_eps)
        self.kv_b_proj = Linear(kv_lora_rank, n_kv_heads * (self.head_dim + self.v_head_dim))
        self.o_proj = Linear(n_heads * self.v_head_dim, dim, init_std=_o_std(n_layers))
        if self.use_gated_attention:
            self.gate = Linear(dim, n_heads * self.v_head_dim)

    def forward(self, x: Tensor, rotary_emb: Tensor, attn_mask: Optional[Tensor] = None, kv_cache=None,
                is_causal: bool = False, fwd: Optional[str] = None) -> Tensor:
        lead = x.shape[:-1]
        nope, rope = self.qk_nope_head_dim, self.qk_rope_head_dim
        if self.q_lora_rank:
            q = self.q_b_proj(self.q_a_norm(self.q_a_proj(x)))
        else:
            q = self.q_proj(x)
        q = q.view(*lead, self.n_heads, self.head_dim)
        kv = self.kv_b_proj(self.kv_norm(self.kv_a_proj(x))).view(*lead, self.n_kv_heads, self.head_dim + self.v_head_dim)
        k_nope, k_rope, v = kv.split((nope, rope, self.v_head_dim), dim=-1)
        q = torch.cat((q[..., :nope], ops.rotary(q[..., nope:], rotary_emb)), dim=-1)
        k = torch.cat((k_nope, ops.rotary(k_rope, rotary_emb)), dim=-1)
        if self.use_qk_norm:
            q, k = self.q_norm(q), self.k_norm(k)
        out = attention(q, k, v.contiguous(), kv_cache, self.layer_id, attn_mask, is_causal, fwd)
        out = out.reshape(*lead, self.dim)
        if self.use_gated_attention:
            out = out * torch.sigmoid(self.gate(x))
        return self.o_proj(out)
