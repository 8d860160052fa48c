"""Load HuggingFace LLaMA-layout checkpoints (config + key names) into this framework's layout.

Behaviour of the reference adapter (``astrai/serialization/hf_adapter.py:32-271``): families llama, mistral,
mixtral, qwen2, qwen2_moe, gemma, gemma2, phi3; biases and DeepSeek MLA checkpoints are rejected; weights are only
renamed (rotary layout is NOT permuted).
"""

from __future__ import annotations

import logging
import re
from typing import Any, Dict, Mapping

import torch

logger = logging.getLogger(__name__)

HF_MODEL_TYPES = frozenset({"llama", "mistral", "mixtral", "qwen2", "qwen2_moe", "gemma", "gemma2", "phi3"})
NATIVE_PREFIXES = ("embed_tokens.", "layers.", "norm.", "lm_head.")

_COPIED_FIELDS = (
    "vocab_size", "hidden_size", "num_hidden_layers", "intermediate_size", "rms_norm_eps", "tie_word_embeddings",
    "max_position_embeddings", "rope_theta", "rope_scaling", "num_attention_heads", "num_key_value_heads",
    "use_qk_norm", "use_gated_attention", "kv_lora_rank", "qk_nope_head_dim", "qk_rope_head_dim", "q_lora_rank",
    "moe_intermediate_size", "shared_expert_intermediate_size", "topk_method", "norm_topk_prob", "moe_aux_loss_coef",
    "decoder_sparse_step", "mlp_only_layers", "neftune_alpha",
)

_L = r"^model\.layers\.(\d+)\."
# (pattern, replacement template, applies-to) ; applies-to: "any", "moe", "dense"
_RULES = [
    (re.compile(_L + r"mlp\.gate\.weight$"), r"layers.\1.mlp.router.weight", "moe"),
    (re.compile(_L + r"mlp\.experts\.(\d+)\.(gate|up|down)_proj\.(weight|bias)$"), r"layers.\1.mlp.routed_experts.\2.\3.\4", "moe"),
    (re.compile(_L + r"mlp\.shared_experts?\.(\d+)\.(gate|up|down)_proj\.(weight|bias)$"), r"layers.\1.mlp.shared_experts.\2.\3.\4", "moe"),
    (re.compile(_L + r"mlp\.(gate|up|down)_proj\.(weight|bias)$"), r"layers.\1.mlp.\2.\3", "dense"),
    (re.compile(_L + r"self_attn\.(q|k|v|o)_proj\.(weight|bias)$"), r"layers.\1.attention.\2_proj.\3", "any"),
    (re.compile(_L + r"self_attn\.(q|k)_norm\.weight$"), r"layers.\1.attention.\2_norm.weight", "any"),
    (re.compile(_L + r"input_layernorm\.weight$"), r"layers.\1.input_norm.weight", "any"),
    (re.compile(_L + r"post_attention_layernorm\.weight$"), r"layers.\1.post_attention_norm.weight", "any"),
    (re.compile(r"^model\.embed_tokens\.weight$"), "embed_tokens.weight", "any"),
    (re.compile(r"^model\.norm\.weight$"), "norm.weight", "any"),
    (re.compile(r"^lm_head\.weight$"), "lm_head.weight", "any"),
]


def looks_like_hf_state_dict(state_dict: Mapping[str, Any]) -> bool:
    markers = ("self_attn.", "input_layernorm", "mlp.experts.")
    return any(k.startswith("model.") or any(m in k for m in markers) for k in state_dict)


def adapt_config(raw: Dict[str, Any]) -> Dict[str, Any]:
    return convert_hf_config(raw) if raw.get("model_type") in HF_MODEL_TYPES else raw


def convert_hf_config(raw: Dict[str, Any]) -> Dict[str, Any]:
    if raw.get("attention_bias") or raw.get("mlp_bias"):
        raise NotImplementedError("attention_bias / mlp_bias checkpoints are not supported; projections are bias-free")
    cfg: Dict[str, Any] = {k: raw[k] for k in _COPIED_FIELDS if k in raw}
    if "use_qk_norm" not in cfg:
        if "qk_norm" in raw:
            cfg["use_qk_norm"] = raw["qk_norm"]
        elif raw.get("model_type") in ("gemma", "gemma2"):
            cfg["use_qk_norm"] = True
    heads = raw.get("num_attention_heads")
    if cfg.get("num_key_value_heads") is None and heads is not None:
        cfg["num_key_value_heads"] = heads
    if raw.get("head_dim") is not None and heads and raw.get("hidden_size"):
        if raw["head_dim"] != raw["hidden_size"] // heads:
            raise NotImplementedError(
                f"HF head_dim={raw['head_dim']} differs from hidden_size/num_attention_heads="
                f"{raw['hidden_size'] // heads}, which this model family derives"
            )
    if "kv_lora_rank" in raw:
        cfg["attn_type"] = "mla"
    n_experts = raw.get("num_local_experts") or raw.get("n_routed_experts")
    if n_experts:
        cfg.update(ffn_type="moe", n_routed_experts=n_experts)
        for src in ("num_experts_per_tok", "n_activated_experts"):
            if src in raw:
                cfg["n_activated_experts"] = raw[src]
        cfg["n_shared_experts"] = raw.get("n_shared_experts", 0)
        if cfg.get("moe_intermediate_size") is None and "intermediate_size" in raw:
            cfg["moe_intermediate_size"] = raw["intermediate_size"]
        dense_first = raw.get("first_k_dense_replace")
        if isinstance(dense_first, int) and dense_first > 0:
            cfg["mlp_only_layers"] = list(range(dense_first))
            cfg["decoder_sparse_step"] = 1
    cfg["model_type"] = "autoregressive_lm"
    return cfg


def _layer_is_dense(config, layer_id: int) -> bool:
    from astrai_b200.models.decoder import ffn_kind

    return ffn_kind(config, layer_id) != "moe"


def convert_hf_weights(state_dict: Mapping[str, Any], config) -> Dict[str, torch.Tensor]:
    """Rename HF keys; native keys pass through; unknown keys are dropped with one warning."""
    if getattr(config, "attn_type", "gqa") == "mla" and any("kv_a_proj_with_mqa" in k for k in state_dict):
        raise NotImplementedError("MLA attention (DeepSeek-V2/V3 kv_a_proj_with_mqa) uses a different KV factorization and cannot be converted")
    moe = getattr(config, "ffn_type", "mlp") == "moe"
    out: Dict[str, torch.Tensor] = {}
    dropped = []
    for key, tensor in state_dict.items():
        if key.startswith(NATIVE_PREFIXES):
            out[key] = tensor
            continue
        target = None
        for pat, template, scope in _RULES:
            m = pat.match(key)
            if not m:
                continue
            if scope == "moe" and not moe:
                continue
            if scope == "dense" and moe and not _layer_is_dense(config, int(m.group(1))):
                continue
            target = m.expand(template)
            break
        if target is None:
            dropped.append(key)
        else:
            out[target] = tensor
    if dropped:
        logger.warning("Dropped %d unmapped HuggingFace weight key(s): %s", len(dropped), ", ".join(sorted(dropped)[:10]))
    return out
