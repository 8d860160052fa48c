"""Pre-norm residual decoder block (reference ``astrai/model/components/decoder_block.py:19-76``)."""

from __future__ import annotations

import dataclasses
from typing import Optional, TypedDict

import torch.nn as nn
from torch import Tensor

from astrai_b200 import ops
from astrai_b200.models.attention import AttnFactory
from astrai_b200.models.ffn import FFNFactory, RouterStats
from astrai_b200.models.layers import RMSNorm


class DecoderOutput(TypedDict):
    hidden_states: Tensor
    aux_loss: Optional[Tensor]
    router_stats: Optional[RouterStats]


def ffn_kind(config, layer_id: int) -> str:
    """Dense or sparse FFN for this layer: ``mlp_only_layers`` and ``decoder_sparse_step`` decide."""
    if config.ffn_type != "moe":
        return config.ffn_type
    if layer_id in (getattr(config, "mlp_only_layers", None) or ()):
        return "mlp"
    step = getattr(config, "decoder_sparse_step", 1)
    if step > 1 and (layer_id + 1) % step != 0:
        return "mlp"
    return "moe"


class DecoderBlock(nn.Module):
    def __init__(self, config, layer_id: int):
        super().__init__()
        kw = dataclasses.asdict(config)
        kw.update(
            dim=config.hidden_size, dim_ffn=config.intermediate_size, n_layers=config.num_hidden_layers,
            n_heads=config.num_attention_heads, n_kv_heads=config.num_key_value_heads, norm_eps=config.rms_norm_eps,
            down_init_std=0.02 / (2 * config.num_hidden_layers) ** 0.5,
        )
        self.layer_id = layer_id
        self.attention = AttnFactory.create(config.attn_type, **kw, layer_id=layer_id)
        self.input_norm = RMSNorm(config.hidden_size, config.rms_norm_eps)
        self.post_attention_norm = RMSNorm(config.hidden_size, config.rms_norm_eps)
        self.mlp = FFNFactory.create(ffn_kind(config, layer_id), **kw)

    def forward(self, x: Tensor, rotary_emb: Tensor, attention_mask: Optional[Tensor] = None, kv_cache=None,
                is_causal: bool = False, fwd: Optional[str] = None, pending: Optional[Tensor] = None,
                defer_residual: bool = False) -> DecoderOutput:
        """``pending``: the FFN output of the block before this one, not yet added to ``x`` - the add then happens inside
        this block's first norm kernel.  ``defer_residual``: return this block's FFN output under ``"pending"`` instead
        of adding it (the caller passes it to the next block, or to the final norm).  A stack of blocks chained this way
        never runs a separate residual-add kernel; without the two arguments the block is ``x + attn(..) + ffn(..)``."""
        if pending is not None:
            x, h0 = self.input_norm(x, residual=pending)
        else:
            h0 = self.input_norm(x)
        attn = self.attention(h0, rotary_emb, attention_mask, kv_cache, is_causal, fwd)
        # residual add and the norm that follows it as one pass over the rows (one kernel on CUDA)
        x, h = ops.add_rms_norm(x, attn, self.post_attention_norm.weight, self.post_attention_norm.norm_eps)
        ffn = self.mlp(h)
        out = {"aux_loss": ffn["aux_loss"], "router_stats": ffn.get("router_stats")}
        if defer_residual:
            out["hidden_states"], out["pending"] = x, ffn["hidden_states"]
        else:
            out["hidden_states"] = x + ffn["hidden_states"]
        return out
