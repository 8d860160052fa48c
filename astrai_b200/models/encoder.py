"""Text-embedding encoder: the decoder trunk without a head, bidirectional by default, pooled to one vector.

Reference: ``astrai/model/encoder.py:16-97`` (pooling ``mean`` (mask-aware) / ``cls`` / ``last``; optional L2
normalisation; a leftover ``lm_head.weight`` in a checkpoint is ignored).
"""

from __future__ import annotations

from typing import Any, Mapping, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch import Tensor

from astrai_b200.config.model_config import EncoderConfig
from astrai_b200.models.automodel import AutoModel, ModelFactory
from astrai_b200.models.decoder import DecoderBlock
from astrai_b200.models.layers import Embedding, RMSNorm, RotaryEmbedding
from astrai_b200.models.lm import _init_module, expand_mask


@ModelFactory.register("embedding")
class EmbeddingEncoder(AutoModel):
    def __init__(self, config: EncoderConfig):
        super().__init__(config)
        self.rotary_embedding = RotaryEmbedding(
            config.hidden_size // config.num_attention_heads, config.max_position_embeddings,
            config.rope_theta if config.rope_theta is not None else 10000, rope_scaling=config.rope_scaling,
        )
        self.embed_tokens = Embedding(config.vocab_size, config.hidden_size, neftune_alpha=config.neftune_alpha)
        self.layers = nn.ModuleList(DecoderBlock(config, i) for i in range(config.num_hidden_layers))
        self.norm = RMSNorm(config.hidden_size, config.rms_norm_eps)
        self.pooling_type = config.pooling_type or "mean"
        self.normalize_embeddings = bool(config.normalize_embeddings)
        self.apply(_init_module)

    def load_state_dict(self, state_dict: Mapping[str, Any], strict=True, assign=False):
        sd = {k: v for k, v in state_dict.items() if k != "lm_head.weight"}
        return super().load_state_dict(sd, strict=strict, assign=assign)

    def pool(self, hidden: Tensor, input_mask: Optional[Tensor]) -> Tensor:
        if self.pooling_type == "cls":
            return hidden[:, 0]
        if self.pooling_type == "last":
            if input_mask is None:
                return hidden[:, -1]
            last = input_mask.sum(dim=1) - 1
            return hidden[torch.arange(hidden.size(0), device=hidden.device), last]
        if input_mask is None:
            return hidden.mean(dim=1)
        m = input_mask.unsqueeze(-1).to(hidden.dtype)
        return (hidden * m).sum(dim=1) / m.sum(dim=1).clamp(min=1.0)

    def forward(self, input_ids: Tensor, input_mask: Optional[Tensor] = None,
                position_ids: Optional[Tensor] = None) -> Tensor:
        if input_ids.ndim != 2:
            raise ValueError("input_ids must be [batch, seq_len]")
        x = self.embed_tokens(input_ids)
        rotary = self.rotary_embedding(x, position_ids)
        mask = expand_mask(input_mask)
        for layer in self.layers:
            x = layer(x, rotary, mask)["hidden_states"]
        pooled = self.pool(self.norm(x), input_mask)
        return F.normalize(pooled, p=2, dim=-1) if self.normalize_embeddings else pooled
