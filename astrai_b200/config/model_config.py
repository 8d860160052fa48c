"""Model architecture configs.

Reference: ``astrai/config/model_config.py:13-178``.  Field names and defaults
are the reference's (they are the ``config.json`` schema of its checkpoints).
``q_lora_rank`` and ``mla_latent_cache`` are additions for the low-rank-query /
latent-cache form of MLA, which the reference does not have; both default to
the reference behaviour.
"""

from typing import Any, Dict, Optional

from pydantic import field_validator
from pydantic.dataclasses import dataclass

from astrai_b200.config.base import BaseConfig, one_of
from astrai_b200.factory import BaseFactory

ATTN_TYPES = ("gqa", "mla")
FFN_TYPES = ("mlp", "moe")
POOLING_TYPES = ("mean", "cls", "last")


class ConfigFactory(BaseFactory[BaseConfig]):
    """``model_type`` -> config class."""

    DEFAULT_TYPE = "autoregressive_lm"

    @classmethod
    def load(cls, raw) -> BaseConfig:
        """The config object for a ``config.json`` dictionary (or the path of such a file), by its ``model_type``."""
        if not isinstance(raw, dict):
            import json

            with open(raw, "r", encoding="utf-8") as fh:
                raw = json.load(fh)
        kind = raw.get("model_type") or cls.DEFAULT_TYPE
        return cls.get_component_class(kind).from_dict(raw)


@dataclass
class BaseModelConfig(BaseConfig):
    model_type: Optional[str] = None
    neftune_alpha: float = 0.0


@dataclass
class _TrunkConfig(BaseModelConfig):
    """Fields shared by the decoder LM and the embedding encoder."""

    vocab_size: Optional[int] = None
    hidden_size: Optional[int] = None
    num_hidden_layers: Optional[int] = None
    rms_norm_eps: Optional[float] = None
    intermediate_size: Optional[int] = None
    max_position_embeddings: Optional[int] = None
    rope_theta: Optional[float] = None
    rope_scaling: Optional[dict] = None
    attn_type: str = "gqa"
    num_attention_heads: Optional[int] = None
    num_key_value_heads: Optional[int] = None
    use_qk_norm: Optional[bool] = None
    use_gated_attention: Optional[bool] = None
    ffn_type: str = "mlp"

    @field_validator("attn_type")
    def _check_attn(cls, v):
        return one_of("attn_type", ATTN_TYPES)(v)

    @field_validator("ffn_type")
    def _check_ffn(cls, v):
        return one_of("ffn_type", FFN_TYPES)(v)

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_attention_heads


@dataclass
@ConfigFactory.register("autoregressive_lm")
class AutoRegressiveLMConfig(_TrunkConfig):
    tie_word_embeddings: Optional[bool] = None
    kv_lora_rank: Optional[int] = None
    qk_nope_head_dim: Optional[int] = None
    qk_rope_head_dim: Optional[int] = None
    q_lora_rank: Optional[int] = None
    v_head_dim: Optional[int] = None
    n_routed_experts: Optional[int] = None
    n_shared_experts: Optional[int] = None
    n_activated_experts: Optional[int] = None
    topk_method: Optional[str] = None
    moe_intermediate_size: Optional[int] = None
    shared_expert_intermediate_size: Optional[int] = None
    norm_topk_prob: bool = True
    decoder_sparse_step: int = 1
    mlp_only_layers: Optional[list[int]] = None
    moe_aux_loss_coef: float = 0.01

    @field_validator("decoder_sparse_step")
    def _check_sparse_step(cls, v):
        if v < 1:
            raise ValueError(f"decoder_sparse_step must be at least 1, got {v}")
        return v

    def to_dict(self):
        d = super().to_dict()
        for extension in ("q_lora_rank", "v_head_dim"):  # fields the reference's config.json does not have
            if d.get(extension) is None:
                d.pop(extension, None)
        return d


@dataclass
@ConfigFactory.register("embedding")
class EncoderConfig(_TrunkConfig):
    pooling_type: Optional[str] = None
    normalize_embeddings: Optional[bool] = None
