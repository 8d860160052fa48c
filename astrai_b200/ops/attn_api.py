"""Functional attention calls under the reference's names (``astrai/extension/ops/attention.py:23-200``).

The reference exposes its kernels one by one (``attn_prefill``, ``attn_decode``, ``attn_paged_decode``) next to the
back-end classes.  Here they are thin front ends of the same operators the models use, so that code written against
those names runs unchanged: dense ``[batch, length, heads, head_dim]`` tensors (the reference's ``BLHD``) go to
:func:`~astrai_b200.ops.attention.dense_attention`, the paged call builds a :class:`~astrai_b200.ops.kv.KVCache` view
and goes to :func:`~astrai_b200.ops.paged_attention.cached_attention`.  Which kernels run is decided there (tcgen05 on a
B200 for the shapes they cover, PyTorch otherwise).
"""

from __future__ import annotations

import enum
from typing import Optional

import torch
from torch import Tensor


class TensorLayout(enum.IntEnum):
    BHLD = 0  # [batch, heads, length, head_dim]
    BLHD = 1  # [batch, length, heads, head_dim]


def _blhd(t: Tensor, layout: TensorLayout) -> Tensor:
    return t if layout == TensorLayout.BLHD else t.transpose(1, 2)


def _dense_mask(mask: Optional[Tensor], q_len: int, kv_len: int, is_causal: bool, device) -> Optional[Tensor]:
    """Boolean ``[B | 1, 1, q_len, kv_len]`` (True = attend) from a 2-D key mask, a 3-D mask and / or causality with the
    queries aligned to the END of the keys (query ``i`` sees keys up to ``kv_len - q_len + i``)."""
    out = None
    if mask is not None:
        out = mask.bool()
        out = out[:, None, None, :] if out.dim() == 2 else out[:, None] if out.dim() == 3 else out
    if is_causal and q_len > 1:
        tri = torch.ones(q_len, kv_len, dtype=torch.bool, device=device).tril(diagonal=kv_len - q_len)[None, None]
        out = tri if out is None else out & tri
    return out


def attn_prefill(q: Tensor, k: Tensor, v: Tensor, mask: Optional[Tensor] = None, is_causal: bool = False,
                 layout: TensorLayout = TensorLayout.BLHD) -> Tensor:
    """Grouped-query attention of ``q_len`` queries over ``kv_len >= q_len`` keys; returns the layout it was given."""
    from astrai_b200.ops.attention import dense_attention

    q, k, v = (_blhd(t, layout) for t in (q, k, v))
    q_len, kv_len = q.shape[1], k.shape[1]
    if mask is None and is_causal and q_len == kv_len:
        out = dense_attention(q, k, v, None, True)  # the flash kernels' own case
    else:
        out = dense_attention(q, k, v, _dense_mask(mask, q_len, kv_len, is_causal, q.device), False)
    return out if layout == TensorLayout.BLHD else out.transpose(1, 2)


def attn_decode(q: Tensor, k: Tensor, v: Tensor, mask: Optional[Tensor] = None, is_causal: bool = False,
                layout: TensorLayout = TensorLayout.BLHD) -> Tensor:
    """One query per row over ``kv_len`` keys (the last key is the query's own position, so causality hides nothing)."""
    if _blhd(q, layout).shape[1] != 1:
        raise ValueError("attn_decode takes exactly one query position per row")
    return attn_prefill(q, k, v, mask, False, layout)


def attn_paged_decode(q: Tensor, k_cache: Tensor, v_cache: Tensor, req_to_token: Tensor, req_pool_indices: Tensor,
                      kv_indptr: Tensor, new_k: Optional[Tensor] = None, new_v: Optional[Tensor] = None,
                      mask: Optional[Tensor] = None, is_causal: bool = False, o_part_buf: Optional[Tensor] = None,
                      ml_part_buf: Optional[Tensor] = None, out_buf: Optional[Tensor] = None) -> Tensor:
    """Decode attention over a flat K / V pool ``[slots, kv_heads, head_dim]``: request ``i`` is row
    ``req_pool_indices[i]`` of the slot table and has ``kv_indptr[i + 1] - kv_indptr[i]`` positions, the last of which is
    the step's own token.  ``new_k`` / ``new_v`` ``[batch, kv_heads, head_dim]`` are stored into that position's slot
    first (when absent, the pool already holds them).  ``q`` and the result are ``[batch, heads, head_dim]``."""
    from astrai_b200.ops.kv import KVCache
    from astrai_b200.ops.paged_attention import cached_attention

    lens = (kv_indptr[1:] - kv_indptr[:-1]).to(torch.long)
    rows = req_pool_indices.to(torch.long)
    loc = req_to_token[rows, lens - 1].to(torch.long)
    if new_k is None or new_v is None:
        new_k, new_v = k_cache[loc], v_cache[loc]
    cache = KVCache(k_buffer=k_cache[None], v_buffer=v_cache[None], req_to_token=req_to_token, req_pool_indices=req_pool_indices,
                    seq_lens=lens.to(req_pool_indices.dtype), out_cache_loc=loc, max_len=int(req_to_token.shape[1]), kv_indptr=kv_indptr)
    out = cached_attention(q, new_k, new_v, cache, 0, mask, True, "decode")
    if out_buf is not None:
        out_buf.copy_(out)
        return out_buf
    return out


def apply_rotary_emb(x: Tensor, freqs_cis: Tensor) -> Tensor:
    """Rotate adjacent pairs of the last dimension of ``x [..., heads, head_dim]`` by the (cos, sin) rows
    ``freqs_cis [..., head_dim / 2, 2]`` (``astrai/extension/backend/rotary.py:36-53``)."""
    from astrai_b200.ops.functional import rotary

    return rotary(x, freqs_cis)


def attn_paged_prefill(q: Tensor, k_cache: Tensor, v_cache: Tensor, req_to_token: Tensor, req_pool_indices: Tensor,
                       kv_indptr: Tensor, qo_indptr: Tensor, q_tile_to_batch: Optional[Tensor] = None,
                       q_tile_to_index: Optional[Tensor] = None, mask: Optional[Tensor] = None, is_causal: bool = True) -> Tensor:
    """Ragged prefill over a flat K / V pool that already holds every key of the batch: request ``i`` has queries
    ``q[qo_indptr[i]:qo_indptr[i + 1]]`` (its LAST positions) and ``kv_indptr[i + 1] - kv_indptr[i]`` keys in row
    ``req_pool_indices[i]`` of the slot table.  The tile maps of the reference's kernel are accepted and not needed (the
    kernels here derive their work list from the offsets)."""
    from astrai_b200.ops.kv import KVCache
    from astrai_b200.ops.paged_attention import cached_attention

    q_ptr, kv_ptr = qo_indptr.tolist(), kv_indptr.tolist()
    q_lens = [b - a for a, b in zip(q_ptr[:-1], q_ptr[1:])]
    kv_lens = [b - a for a, b in zip(kv_ptr[:-1], kv_ptr[1:])]
    rows = req_pool_indices.to(torch.long)
    # the slots of the query positions, request after request: their K / V are rewritten with what the pool holds
    loc = torch.cat([req_to_token[r, n - m:n] for r, m, n in zip(rows.tolist(), q_lens, kv_lens)]).to(torch.long)
    cache = KVCache(k_buffer=k_cache[None], v_buffer=v_cache[None], req_to_token=req_to_token, req_pool_indices=req_pool_indices,
                    seq_lens=torch.tensor(kv_lens, dtype=req_pool_indices.dtype, device=q.device), out_cache_loc=loc,
                    max_len=max(kv_lens), kv_indptr=kv_indptr, qo_indptr=qo_indptr, q_lens=q_lens, kv_lens=kv_lens)
    return cached_attention(q, k_cache[loc], v_cache[loc], cache, 0, mask, is_causal, "prefill")


def repeat_kv(x: Tensor, n_rep: int) -> Tensor:
    """``[..., kv_heads, head_dim]`` -> ``[..., kv_heads * n_rep, head_dim]``: every key / value head repeated for the
    query heads that share it (``astrai/extension/backend/attention.py:244-253``)."""
    return x if n_rep == 1 else x.repeat_interleave(n_rep, dim=-2)


def rotary_emb(x: Tensor, freqs_cis: Tensor) -> Tensor:
    return apply_rotary_emb(x, freqs_cis)


def flash_attn_available() -> bool:
    """Whether the flash-attention kernels can run here: the ones of this package, on a GPU with the extension loaded."""
    from astrai_b200.ops import backend

    return backend.is_available(backend.ATTN_BACKEND.TCGEN05)
