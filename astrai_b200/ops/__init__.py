"""Operator layer: hand-written sm_100a kernels behind differentiable Python front ends."""

from astrai_b200.ops import native, reference
from astrai_b200.ops.attention import dense_attention
from astrai_b200.ops.functional import (
    adamw_,
    assume_loss_grad,
    clip_coef,
    cross_entropy,
    embedding,
    gemm,
    linear,
    linear_cross_entropy,
    linear_token_logprobs,
    qkv_rope,
    rms_norm,
    rotary,
    sumsq,
    swiglu,
    swiglu_fused,
)

__all__ = [
    "adamw_", "assume_loss_grad", "clip_coef", "cross_entropy", "dense_attention", "embedding", "gemm", "linear",
    "linear_cross_entropy", "linear_token_logprobs", "native", "qkv_rope", "reference", "rms_norm", "rotary",
    "sumsq", "swiglu", "swiglu_fused",
]
