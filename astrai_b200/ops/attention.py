"""Attention entry points.

``dense_attention`` serves training and the no-cache forward: q ``[B,S,Hq,D]``, k/v ``[B,L,Hkv,D]``, optional
bool mask (True = attend) or causal flag - the contract of ``astrai/extension/backend/attention.py:256-303``
for ``fwd=None``.  Unmasked and causal calls run on the tcgen05 flash kernels (:mod:`astrai_b200.ops.flash`);
an arbitrary boolean mask goes to the library SDPA kernel.  While a context-parallel context is installed
(:func:`astrai_b200.parallel.context_parallel.init_context_parallel`) causal calls are the sequence-sharded
``ring_attention``.  The packed prefill / paged decode entry points used by the inference engine live in
:mod:`astrai_b200.ops.paged_attention`.
"""

from __future__ import annotations

import os
from typing import Optional

import torch
import torch.nn.functional as F
from torch import Tensor

from astrai_b200.ops import flash, reference

_SDPA_BACKENDS = None


def _use_flash() -> bool:
    """The tcgen05 kernels serve every unmasked / causal call; ``attn_backend("torch_native")`` or
    ``ASTR_BACKEND=torch_native`` selects the library path (comparison baseline; also used for boolean masks)."""
    from astrai_b200.ops import backend

    return backend.get_backend("cuda") is backend.ATTN_BACKEND.TCGEN05


def _sdpa_ctx():
    """Library attention for the dense training path: cuDNN fused attention first, then flash, then the rest."""
    global _SDPA_BACKENDS
    from torch.nn.attention import SDPBackend, sdpa_kernel

    if _SDPA_BACKENDS is None:
        order = os.environ.get("ASTRAI_B200_SDPA", "cudnn,flash,efficient,math").split(",")
        table = {
            "cudnn": SDPBackend.CUDNN_ATTENTION, "flash": SDPBackend.FLASH_ATTENTION,
            "efficient": SDPBackend.EFFICIENT_ATTENTION, "math": SDPBackend.MATH,
        }
        _SDPA_BACKENDS = [table[o] for o in order if o in table]
    return sdpa_kernel(_SDPA_BACKENDS, set_priority=True)


def dense_attention(q: Tensor, k: Tensor, v: Tensor, mask=None, causal: bool = False,
                    scale: Optional[float] = None) -> Tensor:
    """Softmax attention with GQA head sharing; returns ``[B,S,Hq,Dv]``.  ``mask`` is a boolean tensor (True = attend)
    or an :class:`~astrai_b200.ops.segments.AttentionSegments` (causal inside runs of tokens), which runs on the
    variable-length flash kernels."""
    from astrai_b200.ops.segments import AttentionSegments

    if isinstance(mask, AttentionSegments):
        seg = mask
        from astrai_b200.parallel import context_parallel as cpar_

        cp_ = cpar_.get_context()
        if cp_ is not None and cp_.active:
            raise RuntimeError("context parallelism is on: packed-document / padded batches are not sequence-sharded")
        b, s = q.shape[0], q.shape[1]
        if (q.is_cuda and _use_flash() and flash.supported(q, k, v) and k.shape[1] == s
                and (b, s) == (seg.batch, seg.seq_len)):
            cu = seg.cu_seqlens(q.device)
            out = flash.flash_attention_varlen(q.reshape(b * s, *q.shape[2:]), k.reshape(b * s, *k.shape[2:]),
                                               v.reshape(b * s, *v.shape[2:]), cu, cu, seg.max_len, seg.max_len,
                                               causal=True, scale=scale)
            return out.view(b, s, *out.shape[1:])
        mask, causal = seg.to_dense(q.device), False
    from astrai_b200.parallel import context_parallel as cpar

    cp = cpar.get_context()
    if cp is None or not cp.active:
        if not q.is_cuda:
            return reference.attention(q, k, v, mask, causal, scale)
    else:
        # Sequence-sharded training: the local rows are this rank's zig-zag share of the sequence and the keys of the
        # other ranks are fetched inside the attention kernel.  Only plain causal attention is sharded: a call with a
        # mask (packed-document, padding) would silently attend to the local keys only, so it is an error.
        if not causal or mask is not None:
            raise RuntimeError("context parallelism is on: only causal attention without a mask is sequence-sharded "
                               "(use the seq strategy, or switch context parallelism off for this call with "
                               "CPContext.paused())")
        if q.is_cuda and not cpar.supported(q, k, v):
            raise RuntimeError("context parallelism is on, but this attention call is outside what the sharded "
                               "kernels take (bf16, head_dim 64 / 128, local length a multiple of 256)")
        return cpar.ring_attention(q, k, v, scale=scale, ctx=cp, comm=getattr(cp, "comm", "p2p"))
    if _use_flash():
        if mask is None and flash.supported(q, k, v):
            return flash.flash_attention(q, k, v, causal=causal, scale=scale)
        from astrai_b200.ops import backend

        if backend.explicit() and backend._current.get() is not None:
            raise RuntimeError("the tcgen05 attention backend was selected explicitly but does not cover this call "
                               "(boolean mask, or head_dim outside {64, 128})")
    hq, hkv = q.shape[2], k.shape[2]
    qt, kt, vt = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
    with _sdpa_ctx():
        out = F.scaled_dot_product_attention(
            qt, kt, vt, attn_mask=mask, is_causal=causal and mask is None, scale=scale, enable_gqa=hq != hkv
        )
    return out.transpose(1, 2)


def attention(q: Tensor, k: Tensor, v: Tensor, kv_cache=None, layer_id: int = 0, attn_mask: Optional[Tensor] = None,
              is_causal: bool = False, fwd: Optional[str] = None) -> Tensor:
    """Single entry used by the model blocks (signature of the reference's ``attention(...)``,
    ``astrai/extension/backend/attention.py:256-303``).

    ``fwd=None``: dense ``[B,S,H,D]`` tensors, no cache.  ``fwd in {"prefill","decode"}``: packed ``[T,H,D]``
    tensors plus a :class:`~astrai_b200.ops.kv.KVCache`; new K/V are appended to the pool first.
    """
    from astrai_b200.ops import backend

    own = backend.current_custom()
    if own is not None:  # a registered back end that computes attention itself
        return own.forward(q, k, v, kv_cache, layer_id, attn_mask, is_causal, fwd)
    if fwd is None:
        return dense_attention(q, k, v, attn_mask, is_causal)
    from astrai_b200.ops.paged_attention import cached_attention

    return cached_attention(q, k, v, kv_cache, layer_id, attn_mask, is_causal, fwd)
