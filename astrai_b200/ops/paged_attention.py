"""Attention with a KV cache: append this step's K/V to the pool, then attend over the cached prefix + new tokens.

Packed layout: ``q [T, Hq, D]``, ``k / v [T, Hkv, D]`` where the batch is concatenated along ``T``.
* ``fwd="decode"`` (one new token per request): the split-KV paged kernel (``paged_attention.cu``) on CUDA, which also
  stores the step's K / V rows into the pool (no separate append launch);
* ``fwd="prefill"`` (ragged, possibly with a cached prefix): ONE varlen launch of the tcgen05 flash kernel
  (``flash_fwd.cu``, lower-right aligned causal mask) serves every request.  With pages of 8 / 16 / 32 / 64 tokens the
  kernel reads K / V straight from the pool through the slot table; other page sizes (and the contiguous layout's
  page size 1) gather the batch's keys into packed tensors first.  Head dims other than 64 / 128 and explicit masks
  take a per-request SDPA loop.
The CPU statement of both is the same gather + softmax and is what the tests compare against
(semantics of ``TorchNativeBackend`` in the reference, ``astrai/extension/backend/attention.py:443-498``).
"""

from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F
from torch import Tensor

from astrai_b200.ops import flash, native
from astrai_b200.ops.kv import KVCache


def _append(k: Tensor, v: Tensor, cache: KVCache, layer_id: int):
    kb, vb = cache.k_buffer[layer_id], cache.v_buffer[layer_id]
    loc = cache.out_cache_loc.reshape(-1)
    if k.is_cuda and k.dtype == torch.bfloat16 and kb.dtype == torch.bfloat16 and (kb.shape[1] * kb.shape[2]) % 8 == 0:
        native.require()
        torch.ops.astrai_b200.kv_append_(k.contiguous(), v.contiguous(), kb, vb, loc.to(torch.int32))
    else:
        idx = loc.long()
        kb[idx] = k.to(kb.dtype)
        vb[idx] = v.to(vb.dtype)


def _gather_kv(cache: KVCache, layer_id: int, row: int, length: int):
    slots = cache.req_to_token[row, :length].long()
    return cache.k_buffer[layer_id][slots], cache.v_buffer[layer_id][slots]


def _sdpa_one(q: Tensor, k: Tensor, v: Tensor, causal: bool, mask_row: Optional[Tensor] = None) -> Tensor:
    """q [S,Hq,D], k/v [L,Hkv,D]; causal is lower-right aligned (query i sees keys <= L-S+i)."""
    s, l = q.shape[0], k.shape[0]
    hq, hkv = q.shape[1], k.shape[1]
    qt, kt, vt = q.transpose(0, 1)[None], k.transpose(0, 1)[None], v.transpose(0, 1)[None]
    attn_mask = None
    if causal and not (s == l):
        i = torch.arange(s, device=q.device)[:, None]
        j = torch.arange(l, device=q.device)[None, :]
        attn_mask = j <= (l - s + i)
    if mask_row is not None:
        attn_mask = mask_row if attn_mask is None else (attn_mask & mask_row)
    if not q.is_cuda and hq != hkv:
        kt = kt.repeat_interleave(hq // hkv, dim=1)
        vt = vt.repeat_interleave(hq // hkv, dim=1)
        out = F.scaled_dot_product_attention(qt, kt, vt, attn_mask=attn_mask, is_causal=causal and attn_mask is None)
    else:
        out = F.scaled_dot_product_attention(qt, kt, vt, attn_mask=attn_mask, is_causal=causal and attn_mask is None,
                                             enable_gqa=hq != hkv)
    return out[0].transpose(0, 1)


def _lens(cache: KVCache):
    kv = cache.kv_lens if cache.kv_lens is not None else cache.seq_lens.tolist()
    if cache.q_lens is not None:
        return cache.q_lens, kv
    if cache.qo_indptr is not None:
        ptr = cache.qo_indptr.tolist()
        return [b - a for a, b in zip(ptr[:-1], ptr[1:])], kv
    return [1] * len(kv), kv


def _decode_native_ok(q: Tensor, cache: KVCache) -> bool:
    return (
        q.is_cuda and q.dtype == torch.bfloat16 and cache.k_buffer.dtype == torch.bfloat16
        and q.shape[-1] in (32, 64, 128, 256) and cache.decode_o_part is not None and cache.decode_counters is not None
        and q.shape[1] % cache.k_buffer.shape[2] == 0 and 1 <= q.shape[1] // cache.k_buffer.shape[2] <= 8
    )


def cached_attention(q: Tensor, k: Tensor, v: Tensor, kv_cache: KVCache, layer_id: int = 0,
                     attn_mask: Optional[Tensor] = None, is_causal: bool = True, fwd: str = "prefill") -> Tensor:
    if kv_cache is None:
        raise ValueError("inference attention requires a KV cache")
    if q.dim() != 3:
        raise ValueError("packed inference tensors must be [tokens, heads, head_dim]")
    scale = q.shape[-1] ** -0.5
    from astrai_b200.ops import backend as _backend

    native_on = _backend.get_backend(q.device.type) is _backend.ATTN_BACKEND.TCGEN05
    if native_on and fwd == "decode" and attn_mask is None and _decode_native_ok(q, kv_cache):
        # one launch: the step's K / V rows are stored into the pool by the attention kernel itself (the reference fuses
        # its append the same way, csrc/kernels/attention/layout_policies.cuh:221-254)
        b = q.shape[0]
        splits = kv_cache.decode_splits or int(torch.ops.astrai_b200.paged_decode_splits(
            b, kv_cache.k_buffer.shape[2], max(kv_cache.max_len, 1), kv_cache.decode_o_part.shape[2]))
        out = kv_cache.decode_out[:b] if kv_cache.decode_out is not None else torch.empty_like(q)
        torch.ops.astrai_b200.paged_decode_append_(
            q.contiguous(), k.contiguous(), v.contiguous(), kv_cache.k_buffer[layer_id], kv_cache.v_buffer[layer_id],
            kv_cache.req_to_token, kv_cache.req_pool_indices, kv_cache.seq_lens, scale, splits, kv_cache.decode_o_part,
            kv_cache.decode_ml_part, kv_cache.decode_counters, out)
        return out
    _append(k, v, kv_cache, layer_id)
    q_lens, kv_lens = _lens(kv_cache)
    page = getattr(kv_cache, "page_size", 1) or 1
    if (native_on and attn_mask is None and fwd == "prefill" and kv_cache.qo_indptr is not None and page in flash.PAGED_PAGE_SIZES
            and flash.supported(q, kv_cache.k_buffer[layer_id], kv_cache.v_buffer[layer_id])):
        # ragged prefill over the paged pool: the kernel walks the slot table itself (no gathered copy of the keys)
        return flash.flash_attention_paged(q, kv_cache.k_buffer[layer_id], kv_cache.v_buffer[layer_id], kv_cache.qo_indptr,
                                           kv_cache.kv_indptr, kv_cache.req_to_token, kv_cache.req_pool_indices, page,
                                           max(q_lens), causal=True, scale=scale)
    if (native_on and attn_mask is None and fwd == "prefill" and kv_cache.kv_gather_loc is not None and kv_cache.qo_indptr is not None
            and flash.supported(q, kv_cache.k_buffer[layer_id], kv_cache.v_buffer[layer_id])):
        # ragged prefill on the tcgen05 flash kernel: gather this batch's keys / values from the pool (cached prefix
        # included) into packed tensors once, then one varlen launch with lower-right aligned causal masking
        kk = kv_cache.k_buffer[layer_id].index_select(0, kv_cache.kv_gather_loc)
        vv = kv_cache.v_buffer[layer_id].index_select(0, kv_cache.kv_gather_loc)
        return flash.flash_attention_varlen(q, kk, vv, kv_cache.qo_indptr, kv_cache.kv_indptr, max(q_lens), max(kv_lens),
                                            causal=True, scale=scale)
    rows = kv_cache.req_pool_indices.tolist()
    outs, start = [], 0
    for i, (ql, kl) in enumerate(zip(q_lens, kv_lens)):
        kk, vv = _gather_kv(kv_cache, layer_id, rows[i], kl)
        mask_row = None
        if attn_mask is not None:
            mask_row = attn_mask[i].reshape(-1, attn_mask.shape[-1])[..., :kl].bool()
        causal = is_causal or fwd == "decode" or ql > 1
        outs.append(_sdpa_one(q[start:start + ql], kk.to(q.dtype), vv.to(q.dtype), causal and ql > 1, mask_row))
        start += ql
    return torch.cat(outs, dim=0)
