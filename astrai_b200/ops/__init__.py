"""Operator layer: hand-written sm_100a kernels behind differentiable Python front ends."""

from astrai_b200.ops import fp8, native, reference
from astrai_b200.ops.fp8 import DelayedScaling, DynamicScaling, FP8Format, fp8_autocast
from astrai_b200.ops.attention import attention, dense_attention
from astrai_b200.ops.attn_api import (
    TensorLayout, apply_rotary_emb, attn_decode, attn_paged_decode, attn_paged_prefill, attn_prefill, flash_attn_available, repeat_kv,
    rotary_emb,
)
from astrai_b200.ops.backend import (
    ATTN_BACKEND,
    AttentionBackend,
    AttentionBackendFactory,
    CudaBackend,
    FlashAttnBackend,
    Tcgen05Backend,
    TorchNativeBackend,
    attn_backend,
    get_backend,
)
from astrai_b200.ops.native import KERNEL_NAMES, kernel_available as is_available
from astrai_b200.ops.functional import (
    adamw_,
    add_rms_norm,
    assume_loss_grad,
    clip_coef,
    cross_entropy,
    embedding,
    gemm,
    linear,
    linear_cross_entropy,
    loss_denominator,
    linear_token_logprobs,
    qkv_rope,
    rms_norm,
    rotary,
    sumsq,
    swiglu,
    swiglu_fused,
)

__all__ = [
    "adamw_", "add_rms_norm", "apply_rotary_emb", "assume_loss_grad", "attention", "AttentionBackend",
    "AttentionBackendFactory", "ATTN_BACKEND", "attn_backend", "attn_decode", "attn_paged_decode", "attn_paged_prefill",
    "attn_prefill", "clip_coef", "cross_entropy", "CudaBackend", "DelayedScaling", "dense_attention", "DynamicScaling",
    "embedding", "flash_attn_available", "FlashAttnBackend", "fp8", "fp8_autocast", "FP8Format", "gemm", "get_backend",
    "is_available", "KERNEL_NAMES", "linear", "linear_cross_entropy", "linear_token_logprobs", "loss_denominator",
    "native", "qkv_rope", "reference", "repeat_kv", "rms_norm", "rotary", "rotary_emb", "sumsq", "swiglu",
    "swiglu_fused", "Tcgen05Backend", "TensorLayout", "TorchNativeBackend",
]
