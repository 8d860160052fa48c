"""Fixed-address per-step buffers of the inference hot path (CUDA-graph safe).

Same purpose as ``astrai/inference/workspace.py:16-152``: token ids, positions, request rows, lengths, ragged offsets,
write slots and the split-KV decode scratch are allocated once for ``max_batch_size`` and sliced per step.  Host values
are staged through pinned buffers and copied with one async transfer each.
"""

from __future__ import annotations

from typing import List, Sequence

import torch
from torch import Tensor

MAX_SPLITS = 32
Q_TILE_ROWS = 128


class InferenceWorkspace:
    def __init__(self, max_batch_size: int, max_seq_len: int, max_q_heads: int, head_dim: int, device, dtype,
                 n_kv_heads: int = 1, max_prefill_tokens: int = 0):
        self.max_batch_size, self.max_seq_len = max_batch_size, max_seq_len
        self.max_q_heads, self.head_dim = max_q_heads, head_dim
        self.device, self.dtype = torch.device(device), dtype
        b, dev = max_batch_size, self.device
        i32 = dict(dtype=torch.int32, device=dev)
        self.input_ids = torch.zeros(b, dtype=torch.long, device=dev)
        self.position_ids = torch.zeros(b, dtype=torch.long, device=dev)
        self.req_pool_indices = torch.zeros(b, **i32)
        self.seq_lens = torch.zeros(b, dtype=torch.long, device=dev)
        self.kv_indptr = torch.zeros(b + 1, **i32)
        self.qo_indptr = torch.zeros(b + 1, **i32)
        self.inc = torch.arange(b + 1, **i32)
        self.out_cache_loc = torch.zeros(max(b, max_prefill_tokens), **i32)
        tiles = b * (-(-max_seq_len // Q_TILE_ROWS))
        self.q_tile_to_batch = torch.zeros(tiles, **i32)
        self.q_tile_to_index = torch.zeros(tiles, **i32)
        self.arange = torch.arange(max_seq_len, device=dev)
        self.input_mask = torch.zeros((b, 1, max_seq_len), dtype=torch.bool, device=dev)
        self.decode_o_part = torch.zeros((b, max_q_heads, MAX_SPLITS, head_dim), dtype=torch.float32, device=dev)
        self.decode_ml_part = torch.zeros((b, max_q_heads, MAX_SPLITS, 2), dtype=torch.float32, device=dev)
        self.decode_out = torch.zeros((b, max_q_heads, head_dim), dtype=dtype, device=dev)
        self.decode_counters = torch.zeros(b * max(n_kv_heads, 1), dtype=torch.int32, device=dev)
        pin = dev.type == "cuda"
        # Pinned staging ring: an async copy reads its source later, in stream order, so a slot must not be reused
        # while its copy may still be queued.  The scheduler synchronises once per step (it reads the sampled
        # tokens), and one step issues far fewer than RING puts.
        self._stage_long = [torch.zeros(b, dtype=torch.long, pin_memory=pin) for _ in range(self.RING)]
        self._stage_int = [torch.zeros(max(b, max_prefill_tokens) + b + 2, dtype=torch.int32, pin_memory=pin)
                           for _ in range(self.RING)]
        self._flip = 0

    RING = 32

    def _next(self):
        self._flip = (self._flip + 1) % self.RING
        return self._stage_long[self._flip], self._stage_int[self._flip]

    def put_long(self, dst: Tensor, values: Sequence[int]) -> Tensor:
        """Copy host ints into the first ``len(values)`` entries of a long device buffer."""
        n = len(values)
        stage, _ = self._next()
        stage[:n] = torch.as_tensor(values, dtype=torch.long)
        dst[:n].copy_(stage[:n], non_blocking=True)
        return dst[:n]

    def put_int(self, dst: Tensor, values) -> Tensor:
        vals = torch.as_tensor(values, dtype=torch.int32).reshape(-1)
        n = vals.numel()
        _, stage = self._next()
        if n > stage.numel():
            dst_new = vals.to(self.device)
            return dst_new
        stage[:n] = vals
        if n > dst.numel():
            return stage[:n].to(self.device, non_blocking=True)
        dst[:n].copy_(stage[:n], non_blocking=True)
        return dst[:n]

    def fill_input_ids(self, ids: List[int]) -> Tensor:
        return self.put_long(self.input_ids, ids)

    def decode_mask(self, position_ids: Tensor, total_len: int) -> Tensor:
        b = position_ids.size(0)
        out = self.input_mask[:b, :, :total_len]
        torch.ge(position_ids[:, None, None], self.arange[:total_len], out=out)
        return out
