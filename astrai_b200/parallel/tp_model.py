"""Tensor-parallel form of the decoder: attention heads and FFN columns sharded over the ranks of one block,
activations between the layers sharded along the token axis (sequence parallelism).

``shard_model_`` rewrites an :class:`~astrai_b200.models.lm.AutoRegressiveLM` in place:

* every ``GQA`` block becomes a :class:`TPAttention` (this rank's query / key / value heads, the matching columns of
  ``o_proj``) and every dense ``MLP`` a :class:`TPMLP` (this rank's ``gate`` / ``up`` rows and ``down`` columns);
* embedding, norms and ``lm_head`` stay replicated and work on this rank's ``tokens / tp`` rows only;
* the model's ``forward`` keeps its signature but returns ``hidden_states`` / ``logits`` of the local rows
  ``[tokens / tp, ...]``: rank ``r`` owns rows ``[r * T/tp, (r+1) * T/tp)`` of the flattened ``[B*S]`` token axis.

Inside a block: ``all-gather -> q|k|v GEMM`` (one fused kernel), attention on the local heads over the full sequence,
``o_proj GEMM -> reduce-scatter`` (one fused kernel); the FFN is the same pair around SwiGLU.  The collectives are
those of :mod:`astrai_b200.parallel.tensor_parallel` (``comm="p2p"``: fused peer-memory kernels, ``"nccl"``: library
collectives around the plain GEMM, also the CPU path).

``gather_state_dict`` undoes the sharding for checkpoints: the saved file has the reference's unsharded keys and shapes
(``astrai/serialization/checkpoint.py:152-166``).  The reference has no tensor parallelism
(``scripts/tools/train.py:513-519`` parses ``--tp_size`` and drops it).
"""

from __future__ import annotations

import types
from typing import Dict, Optional

import torch
import torch.distributed as dist
import torch.nn as nn
from torch import Tensor

from astrai_b200 import ops
from astrai_b200.models.layers import Linear, RMSNorm
from astrai_b200.ops.attention import attention
from astrai_b200.parallel.tensor_parallel import _ColumnParallelFn, _RowParallelFn


class _Shape:
    """Batch and sequence length of the forward pass in flight (the blocks only see ``[tokens / tp, dim]``)."""

    batch = 1
    seq = 1


def _linear_from(weight: Tensor) -> Linear:
    lin = Linear(weight.shape[1], weight.shape[0])
    lin.weight = nn.Parameter(weight.detach().clone().contiguous())
    return lin


class TPAttention(nn.Module):
    def __init__(self, src, tp_size: int, tp_rank: int, comm: str):
        super().__init__()
        if type(src).__name__ != "GQA":
            raise NotImplementedError("tensor parallelism covers grouped-query attention blocks")
        if src.use_gated_attention:
            raise NotImplementedError("tensor parallelism does not cover the sigmoid output gate")
        if src.n_heads % tp_size or src.n_kv_heads % tp_size:
            raise ValueError(f"{src.n_heads} query / {src.n_kv_heads} kv heads do not divide over {tp_size} ranks")
        self.tp_size, self.tp_rank, self.comm = tp_size, tp_rank, comm
        self.dim, self.head_dim, self.layer_id = src.dim, src.head_dim, src.layer_id
        self.n_heads, self.n_kv_heads = src.n_heads // tp_size, src.n_kv_heads // tp_size
        self.use_qk_norm = src.use_qk_norm
        d = self.head_dim
        qs = slice(tp_rank * self.n_heads * d, (tp_rank + 1) * self.n_heads * d)
        ks = slice(tp_rank * self.n_kv_heads * d, (tp_rank + 1) * self.n_kv_heads * d)
        self.q_proj = _linear_from(src.q_proj.weight[qs])
        self.k_proj = _linear_from(src.k_proj.weight[ks])
        self.v_proj = _linear_from(src.v_proj.weight[ks])
        self.o_proj = _linear_from(src.o_proj.weight[:, qs])
        if self.use_qk_norm:
            self.q_norm, self.k_norm = src.q_norm, src.k_norm
        self.fused_qkv = None  # set by the flat-buffer engine: q|k|v rows back to back, with .main_grad

    def _qkv_weight(self) -> Tensor:
        if self.fused_qkv is not None:
            return self.fused_qkv
        return torch.cat([self.q_proj.weight, self.k_proj.weight, self.v_proj.weight], dim=0)

    def forward(self, x: Tensor, rotary_emb: Tensor, attn_mask: Optional[Tensor] = None, kv_cache=None,
                is_causal: bool = False, fwd: Optional[str] = None) -> Tensor:
        if fwd is not None:
            raise NotImplementedError("the tensor-parallel blocks are a training form (no KV cache)")
        b, s, hq, hkv, d = _Shape.batch, _Shape.seq, self.n_heads, self.n_kv_heads, self.head_dim
        qkv = _ColumnParallelFn.apply(x, self._qkv_weight(), self.comm)          # [B*S, (hq + 2 hkv) * d]
        q, k, v = ops.qkv_rope(qkv, rotary_emb.reshape(b * s, d // 2, 2), hq, hkv, d)
        q, k, v = q.view(b, s, hq, d), k.view(b, s, hkv, d), v.view(b, s, hkv, d)
        if self.use_qk_norm:
            q, k = self.q_norm(q), self.k_norm(k)
        out = attention(q, k, v, None, self.layer_id, attn_mask, is_causal, None).reshape(b * s, hq * d)
        return _RowParallelFn.apply(out, self.o_proj.weight, self.comm)          # [B*S / tp, dim]


class TPMLP(nn.Module):
    def __init__(self, src, tp_size: int, tp_rank: int, comm: str):
        super().__init__()
        ffn = src.gate.weight.shape[0]
        if ffn % tp_size:
            raise ValueError(f"FFN width {ffn} does not divide over {tp_size} ranks")
        self.tp_size, self.tp_rank, self.comm = tp_size, tp_rank, comm
        rows = slice(tp_rank * ffn // tp_size, (tp_rank + 1) * ffn // tp_size)
        self.gate = _linear_from(src.gate.weight[rows])
        self.up = _linear_from(src.up.weight[rows])
        self.down = _linear_from(src.down.weight[:, rows])
        self.fused_gate_up = None  # set by the flat-buffer engine: gate rows then up rows

    def forward(self, x: Tensor):
        w = self.fused_gate_up
        if w is None:
            w = torch.cat([self.gate.weight, self.up.weight], dim=0)
        gu = _ColumnParallelFn.apply(x, w, self.comm)                              # [B*S, 2 * ffn / tp]
        h = ops.swiglu_fused(gu)
        return {"hidden_states": _RowParallelFn.apply(h, self.down.weight, self.comm), "aux_loss": None, "router_stats": None}


def _tp_forward(self, input_ids: Tensor, input_mask: Optional[Tensor] = None, kv_cache=None,
                position_ids: Optional[Tensor] = None, fwd: Optional[str] = None, return_logits: bool = True):
    """Training forward of the sharded model: full ``input_ids [B, S]`` in, this rank's token rows out."""
    from astrai_b200.models.lm import expand_mask

    if fwd is not None or kv_cache is not None:
        raise NotImplementedError("the tensor-parallel model is a training form (no KV cache)")
    if input_ids.ndim != 2:
        raise ValueError("training input_ids must be [batch, seq_len]")
    tp, r = self._tp_size, self._tp_rank
    b, s = input_ids.shape
    total = b * s
    if total % tp:
        raise ValueError(f"{total} tokens do not divide over {tp} tensor-parallel ranks")
    local = total // tp
    _Shape.batch, _Shape.seq = b, s
    x = self.embed_tokens(input_ids.reshape(-1)[r * local:(r + 1) * local].unsqueeze(0)).squeeze(0)  # [T/tp, dim]
    if position_ids is None:
        position_ids = torch.arange(s, device=input_ids.device).expand(b, -1)
    rotary = self.rotary_embedding.freqs_cis[position_ids]  # [B, S, d/2, 2]: attention sees every token of the batch
    mask = expand_mask(input_mask)
    causal = mask is None
    pending = None
    for layer in self.layers:
        out = layer(x, rotary, mask, None, causal, None, pending=pending, defer_residual=True)
        x, pending = out["hidden_states"], out["pending"]
    _, hidden = self.norm(x, residual=pending)
    out = {"hidden_states": hidden}
    if return_logits:
        out["logits"] = self.lm_head(hidden)
    return out


def shard_model_(model: nn.Module, tp_size: int, tp_rank: int, comm: str = "p2p") -> nn.Module:
    """Replace attention and dense FFN blocks by their tensor-parallel forms (in place) and bind the sharded forward."""
    if getattr(model.config, "ffn_type", "mlp") != "mlp" or getattr(model.config, "attn_type", "gqa") != "gqa":
        raise NotImplementedError("tensor parallelism covers dense GQA decoders; use expert parallelism for MoE models")
    for layer in model.layers:
        layer.attention = TPAttention(layer.attention, tp_size, tp_rank, comm)
        layer.mlp = TPMLP(layer.mlp, tp_size, tp_rank, comm)
    model._tp_size, model._tp_rank = tp_size, tp_rank
    model.forward = types.MethodType(_tp_forward, model)
    return model


SHARDED_DIM = {"q_proj": 0, "k_proj": 0, "v_proj": 0, "gate": 0, "up": 0, "o_proj": 1, "down": 1}


def is_sharded(name: str) -> bool:
    """True for the parameters that differ between the ranks of a tensor-parallel block (by parameter name)."""
    parts = name.split(".")
    return len(parts) >= 2 and parts[-1] == "weight" and parts[-2] in SHARDED_DIM and ("attention" in parts or "mlp" in parts)


def gather_state_dict(model: nn.Module, group=None, dst_only: bool = True) -> Optional[Dict[str, Tensor]]:
    """The unsharded state dict (reference key names and shapes).  Collective over the tensor-parallel group; the
    result is returned on the group's first rank (``None`` elsewhere) unless ``dst_only`` is false."""
    tp = model._tp_size
    first = dist.get_rank(group) == 0 if (dist.is_initialized() and tp > 1) else True
    out: Dict[str, Tensor] = {}
    for name, t in model.state_dict().items():
        if tp > 1 and is_sharded(name):
            dim = SHARDED_DIM[name.split(".")[-2]]
            parts = [torch.empty_like(t) for _ in range(tp)]
            dist.all_gather(parts, t.contiguous(), group=group)
            t = torch.cat(parts, dim=dim)
        if first or not dst_only:
            out[name] = t
    return out if (first or not dst_only) else None
