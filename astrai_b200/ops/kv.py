"""The plain struct handed to the model for KV-cache I/O during inference.

Field names follow the reference's ``KVCache`` (``astrai/inference/cache/buffer.py:73-96``) so that its call sites read
the same: K/V pools ``[layers, slots, kv_heads, head_dim]``, a ``req_to_token`` table mapping (request row, position)
to a slot, per-batch request rows / lengths / write slots, ragged offsets for packed prefill, and decode scratch.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

from torch import Tensor


@dataclass
class KVCache:
    k_buffer: Tensor
    v_buffer: Tensor
    req_to_token: Tensor
    req_pool_indices: Tensor
    seq_lens: Tensor
    out_cache_loc: Tensor
    max_len: int = 0
    kv_indptr: Optional[Tensor] = None
    qo_indptr: Optional[Tensor] = None
    q_tile_to_batch: Optional[Tensor] = None
    q_tile_to_index: Optional[Tensor] = None
    decode_o_part: Optional[Tensor] = None
    decode_ml_part: Optional[Tensor] = None
    decode_out: Optional[Tensor] = None
    decode_counters: Optional[Tensor] = None
    # host copies of the ragged shape, so the prefill path never reads lengths back from the device
    q_lens: Optional[List[int]] = None
    kv_lens: Optional[List[int]] = None
    decode_splits: int = 0
    # prefill: slot of every cached + new key of the batch, request after request (the gather index of the flash path)
    kv_gather_loc: Optional[Tensor] = None
    # tokens per page of the pool (1: slots are not grouped into pages); 8 / 16 / 32 / 64 let prefill read the pool in place
    page_size: int = 1
