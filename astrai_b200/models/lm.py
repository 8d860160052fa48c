"""Decoder-only language model.

Forward contract (reference ``astrai/model/transformer.py:102-152``):
* ``fwd=None``: ``input_ids [B,S]``, no cache -> ``logits [B,S,V]``.  No mask = causal; a 2-D ``[B,S]`` mask is a
  key-padding mask and the pass is then NOT causal (reference quirk, kept); 3-D / 4-D bool masks are used as given.
* ``fwd in {"prefill","decode"}``: packed ``input_ids [T]`` + ``position_ids [T]`` + KV cache -> ``logits [T,V]``.
Output dict: ``logits``, ``hidden_states`` and, for MoE models, ``aux_loss`` (mean over MoE layers) and
``router_stats``.  ``return_logits=False`` skips the vocabulary projection so that a fused
projection + loss (``ops.linear_cross_entropy``) can consume ``hidden_states`` without ``[T,V]`` logits.
"""

from __future__ import annotations

from typing import Any, Dict, Mapping, Optional

import torch
import torch.nn as nn
from torch import Tensor

from astrai_b200.utils import trace
from astrai_b200.config.model_config import AutoRegressiveLMConfig
from astrai_b200.models.automodel import AutoModel, ModelFactory
from astrai_b200.models.decoder import DecoderBlock
from astrai_b200.models.layers import Embedding, Linear, RMSNorm, RotaryEmbedding


def expand_mask(mask: Optional[Tensor]) -> Optional[Tensor]:
    """[B,S] -> [B,1,1,S] (key padding); [B,S,S] -> [B,1,S,S]; 4-D unchanged."""
    if mask is None or not isinstance(mask, Tensor) or mask.dim() == 4:
        return mask  # run boundaries (AttentionSegments) travel to the attention op as they are
    return mask[:, None, None, :] if mask.dim() == 2 else mask[:, None]


process_attention_mask = expand_mask  # the reference's name (``astrai/model/transformer.py:17-26``)


def _init_module(m: nn.Module):
    if hasattr(m, "reset_parameters"):
        m.reset_parameters()


@ModelFactory.register("autoregressive_lm")
class AutoRegressiveLM(AutoModel):
    supports_fused_head = True  # forward(..., return_logits=False) feeds a fused projection + loss

    def __init__(self, config: AutoRegressiveLMConfig):
        super().__init__(config)
        rope_dim = config.qk_rope_head_dim if config.attn_type == "mla" else config.hidden_size // config.num_attention_heads
        self.rotary_embedding = RotaryEmbedding(
            rope_dim, config.max_position_embeddings,
            config.rope_theta if config.rope_theta is not None else 10000, rope_scaling=config.rope_scaling,
        )
        self.embed_tokens = Embedding(config.vocab_size, config.hidden_size, neftune_alpha=config.neftune_alpha)
        self.layers = nn.ModuleList(DecoderBlock(config, i) for i in range(config.num_hidden_layers))
        self.norm = RMSNorm(config.hidden_size, config.rms_norm_eps)
        self.lm_head = Linear(config.hidden_size, config.vocab_size)
        if config.tie_word_embeddings is True:
            self.lm_head.weight = self.embed_tokens.weight
        self.apply(_init_module)

    @property
    def tied(self) -> bool:
        return self.config.tie_word_embeddings is True

    # -- state dict: a tied head is stored once, under the embedding key ---------------------------------------
    def load_state_dict(self, state_dict: Mapping[str, Any], strict=True, assign=False):
        sd = dict(state_dict)
        emb, head = "embed_tokens.weight", "lm_head.weight"
        if emb in sd and (self.tied or head not in sd):
            sd[head] = sd[emb] if self.tied else sd[emb].clone()
        return super().load_state_dict(sd, strict, assign)

    def state_dict(self, *args, destination=None, prefix="", keep_vars=False):
        sd = super().state_dict(*args, destination=destination, prefix=prefix, keep_vars=keep_vars)
        if self.tied:
            sd.pop(prefix + "lm_head.weight", None)
        return sd

    def forward(self, input_ids: Tensor, input_mask: Optional[Tensor] = None, kv_cache=None,
                position_ids: Optional[Tensor] = None, fwd: Optional[str] = None,
                return_logits: bool = True) -> Dict[str, Tensor]:
        if fwd is None:
            if input_ids.ndim != 2:
                raise ValueError("training input_ids must be [batch, seq_len]")
            if kv_cache is not None:
                raise ValueError("training forward does not accept a KV cache")
        elif fwd in ("prefill", "decode"):
            if input_ids.ndim != 1:
                raise ValueError("inference input_ids must be packed [tokens]")
            if kv_cache is None:
                raise ValueError("inference forward requires a KV cache")
        else:
            raise ValueError(f"unsupported forward mode: {fwd}")

        x = self.embed_tokens(input_ids)
        rotary = self.rotary_embedding(x, position_ids)
        mask = expand_mask(input_mask)
        causal = mask is None
        aux, stats = [], []
        pending = None  # FFN output of the previous block: added inside the next norm kernel, never on its own
        for i, layer in enumerate(self.layers):
            if trace.enabled():
                with trace.range(f"layer{i}"):
                    out = layer(x, rotary, mask, kv_cache, causal, fwd, pending=pending, defer_residual=True)
            else:
                out = layer(x, rotary, mask, kv_cache, causal, fwd, pending=pending, defer_residual=True)
            x, pending = out["hidden_states"], out["pending"]
            if out.get("router_stats") is not None:
                aux.append(out["aux_loss"])
                stats.append(out["router_stats"])
        if pending is not None:
            _, hidden = self.norm(x, residual=pending)  # through the module: wrappers hook its call to ready the weight
        else:
            hidden = self.norm(x)
        result: Dict[str, Any] = {"hidden_states": hidden}
        if return_logits:
            result["logits"] = self.lm_head(hidden)
        if aux:
            result["aux_loss"] = torch.stack(aux).mean()
            result["router_stats"] = stats
        return result
