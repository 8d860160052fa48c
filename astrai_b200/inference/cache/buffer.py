"""Physical KV storage: the K/V pools and the request -> slot table.

Same roles as ``astrai/inference/cache/buffer.py:19-96``.  The table keeps a host mirror: slot indices are computed on
the host and shipped to the device in one copy per request (prefill) or per new page (decode) instead of one device
write per token.
"""

from __future__ import annotations

import threading
from typing import List, Optional

import torch

from astrai_b200.ops.kv import KVCache  # noqa: F401  (re-exported)


class ReqToTokenPool:
    def __init__(self, size: int, max_context_len: int, device):
        self.size, self.max_context_len = size, max_context_len
        self.device = torch.device(device)
        self.req_to_token = torch.zeros((size, max_context_len), dtype=torch.int32, device=self.device)
        self.host = torch.zeros((size, max_context_len), dtype=torch.int32)
        if self.device.type == "cuda":
            self.host = self.host.pin_memory()
        self.free_slots: List[int] = list(range(size))
        self._lock = threading.Lock()

    def alloc(self, num_reqs: int) -> Optional[List[int]]:
        with self._lock:
            if num_reqs > len(self.free_slots):
                return None
            taken, self.free_slots = self.free_slots[:num_reqs], self.free_slots[num_reqs:]
            return taken

    def free(self, req_indices: List[int]):
        with self._lock:
            self.free_slots.extend(req_indices)

    def write_row(self, req_idx: int, begin: int, values: torch.Tensor):
        """Set ``table[req_idx, begin:begin+len(values)]`` on host and device (one async copy)."""
        end = begin + values.numel()
        self.host[req_idx, begin:end] = values
        self.req_to_token[req_idx, begin:end].copy_(self.host[req_idx, begin:end], non_blocking=True)

    def write(self, indices, values):
        self.req_to_token[indices] = values


class KVStorage:
    def __init__(self, size: int, n_layers: int, n_kv_heads: int, head_dim: int, device, dtype):
        self.size = size
        self.k_buffer = torch.zeros((n_layers, size, n_kv_heads, head_dim), device=device, dtype=dtype)
        self.v_buffer = torch.zeros((n_layers, size, n_kv_heads, head_dim), device=device, dtype=dtype)
