"""KV cache orchestration: ``PagePool`` (buffers + table + allocation strategy + per-step binding) and
``TaskCacheManager`` (task id -> slots).

Behaviour of the reference (``astrai/inference/cache/pool.py:50-382``) with two deliberate differences: paged mode with
16-token pages and the radix prefix index is the DEFAULT (the reference defaults to contiguous rows and needs a
hand-built pool for paging), and per-step metadata is assembled from the host mirror of the table instead of device
gathers.  Decode metadata is updated in place (``seq_lens += 1``) when the same ordered task set advances by exactly
one token, which keeps CUDA-graph replay valid.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

import torch

from astrai_b200.inference.cache.buffer import KVCache, KVStorage, ReqToTokenPool
from astrai_b200.inference.cache.strategy import (
    AllocationStrategy, Allocator, ContiguousStrategy, PagedStrategy, RadixCache, TaskCacheState,
)
from astrai_b200.inference.workspace import Q_TILE_ROWS, InferenceWorkspace

DEFAULT_PAGE_SIZE = 16


def page_hash(token_ids: List[int], page_idx: int, page_size: int, parent_hash: int = 0) -> int:
    h = parent_hash
    for tok in token_ids[page_idx * page_size:(page_idx + 1) * page_size]:
        h = (h * 31 + tok) & 0xFFFFFFFFFFFFFFFF
    return h


@dataclass
class _BindState:
    sig: tuple
    seq_lens: List[int]


class PagePool:
    def __init__(self, n_layers: int, n_kv_heads: int, head_dim: int, max_batch_size: int, max_seq_len: int, device,
                 dtype, page_size: int = 1, n_tokens: Optional[int] = None):
        self.page_size, self.max_batch_size, self.max_seq_len = page_size, max_batch_size, max_seq_len
        self.device, self.dtype = torch.device(device), dtype
        self.n_layers, self.n_kv_heads, self.head_dim = n_layers, n_kv_heads, head_dim
        self.contiguous = n_tokens is None
        self.n_tokens = max_batch_size * max_seq_len if self.contiguous else (n_tokens // page_size) * page_size
        if self.n_tokens > torch.iinfo(torch.int32).max:
            raise ValueError("KV cache token count exceeds the int32 slot index limit")
        self._storage = KVStorage(self.n_tokens, n_layers, n_kv_heads, head_dim, self.device, dtype)
        self._req_pool = ReqToTokenPool(max_batch_size, max_seq_len, self.device)
        if self.contiguous:
            rows = torch.arange(max_batch_size * max_seq_len, dtype=torch.int32).view(max_batch_size, max_seq_len)
            self._req_pool.host.copy_(rows)
            self._req_pool.req_to_token.copy_(rows)
            self._strategy: AllocationStrategy = ContiguousStrategy()
            self.allocator = self.prefix = None
        else:
            self.allocator = Allocator(self.n_tokens // page_size)
            self.prefix = RadixCache(page_size) if page_size > 1 else None
            if self.prefix is not None:
                self.allocator.on_evict = self.prefix.evict
            self._strategy = PagedStrategy(self.allocator, self.prefix, page_size, self._req_pool, self.device)

    @classmethod
    def for_model(cls, config, max_batch_size: int, max_seq_len: int, device, dtype, page_size: int = DEFAULT_PAGE_SIZE,
                  n_tokens: Optional[int] = None, paged: bool = True) -> "PagePool":
        """Pool sized for a model config; paged with a radix prefix index unless ``paged=False``."""
        head_dim = config.hidden_size // config.num_attention_heads
        if paged and n_tokens is None:
            n_tokens = max_batch_size * (-(-max_seq_len // page_size)) * page_size
        return cls(config.num_hidden_layers, config.num_key_value_heads, head_dim, max_batch_size, max_seq_len, device,
                   dtype, page_size=page_size if paged else 1, n_tokens=n_tokens if paged else None)

    strategy = property(lambda self: self._strategy)
    req_pool = property(lambda self: self._req_pool)
    storage = property(lambda self: self._storage)

    def bind_tasks(self, req_indices: List[int], seq_lens: List[int], workspace: InferenceWorkspace, device=None,
                   start_pos: Optional[int] = None, incremental: bool = False,
                   start_positions: Optional[List[int]] = None) -> KVCache:
        """Per-step ``KVCache`` for a batch.  ``start_pos`` (or per-request ``start_positions``) selects prefill
        (query = positions ``[start, len)``); ``None`` selects decode (query = the last position)."""
        ws, b = workspace, len(req_indices)
        host = self._req_pool.host
        if incremental:
            ws.seq_lens[:b] += 1
            ws.kv_indptr[: b + 1] += ws.inc[: b + 1]
        else:
            ws.put_int(ws.req_pool_indices, req_indices)
            ws.put_long(ws.seq_lens, seq_lens)
            ws.put_int(ws.kv_indptr, [0] + torch.tensor(seq_lens).cumsum(0).tolist())
        rows, lens_t, kv_indptr = ws.req_pool_indices[:b], ws.seq_lens[:b], ws.kv_indptr[: b + 1]
        prefill = start_pos is not None or start_positions is not None
        if prefill:
            starts = start_positions if start_positions is not None else [start_pos] * b
            q_lens = [n - s for n, s in zip(seq_lens, starts)]
            if any(q <= 0 for q in q_lens):
                raise ValueError("prefill sequence lengths must exceed start_pos")
            loc = torch.cat([host[r, s:n] for r, s, n in zip(req_indices, starts, seq_lens)])
            out_cache_loc = ws.put_int(ws.out_cache_loc, loc)
            qo = ws.put_int(ws.qo_indptr, [0] + torch.tensor(q_lens).cumsum(0).tolist())
            tb, ti = [], []
            for i, q in enumerate(q_lens):
                n = -(-q // Q_TILE_ROWS)
                tb += [i] * n
                ti += list(range(n))
            tile_b, tile_i = ws.put_int(ws.q_tile_to_batch, tb), ws.put_int(ws.q_tile_to_index, ti)
            gather = None
            in_place = not self.contiguous and self.page_size in (8, 16, 32, 64)  # the prefill kernel walks the table itself
            if self.device.type == "cuda" and not in_place:  # one index for "all keys of the batch": gathered once per layer
                gather = torch.cat([host[r, :n] for r, n in zip(req_indices, seq_lens)]).to(torch.int64).to(self.device, non_blocking=True)
            return KVCache(self._storage.k_buffer, self._storage.v_buffer, self._req_pool.req_to_token, rows, lens_t,
                           out_cache_loc, max(seq_lens), kv_indptr, qo, tile_b, tile_i, q_lens=q_lens, kv_lens=list(seq_lens),
                           kv_gather_loc=gather, page_size=1 if self.contiguous else self.page_size)
        # slot of every request's newest position: one gather over the host table (a Python loop over the requests costs
        # more than the rest of the step's bookkeeping at large batch sizes)
        loc = host[torch.as_tensor(req_indices, dtype=torch.long), torch.as_tensor(seq_lens, dtype=torch.long) - 1]
        out_cache_loc = ws.put_int(ws.out_cache_loc, loc)
        ws.qo_indptr[: b + 1].copy_(ws.inc[: b + 1])
        max_len = max(seq_lens)
        splits = 0
        if self.device.type == "cuda":
            base = max(b * self.n_kv_heads, 1)
            splits = max(1, min(148 * 2 // base, -(-max_len // 128), ws.decode_o_part.shape[2]))  # one wave of 2 CTAs per SM
        return KVCache(self._storage.k_buffer, self._storage.v_buffer, self._req_pool.req_to_token, rows, lens_t,
                       out_cache_loc, max_len, kv_indptr, ws.qo_indptr[: b + 1], None, None, ws.decode_o_part,
                       ws.decode_ml_part, ws.decode_out, ws.decode_counters, q_lens=[1] * b, kv_lens=list(seq_lens),
                       decode_splits=splits)


class TaskCacheManager:
    def __init__(self, pool: PagePool):
        self._pool, self._strategy, self._req_pool = pool, pool.strategy, pool.req_pool
        self._max_seq_len = pool.max_seq_len
        self._states: Dict[str, TaskCacheState] = {}
        self._bind_state: Optional[_BindState] = None
        self._bind_was_steady = False

    def task_alloc(self, task_id: str, prompt_ids: List[int]) -> bool:
        self._bind_state = None
        rows = self._req_pool.alloc(1)
        if rows is None:
            return False
        state = TaskCacheState(req_idx=rows[0])
        self._states[task_id] = state
        if not self._strategy.alloc(state, prompt_ids):
            self._strategy.free(state)
            self._req_pool.free([state.req_idx])
            self._states.pop(task_id, None)
            return False
        self._strategy.write_indices(state, prompt_ids)
        state.length = len(prompt_ids)
        return True

    def task_free(self, task_id: str):
        self._bind_state = None
        state = self._states.pop(task_id, None)
        if state is not None:
            self._strategy.free(state)
            self._req_pool.free([state.req_idx])

    def task_extend(self, task_id: str, pos: int) -> bool:
        state = self._states.get(task_id)
        if state is None or pos >= self._max_seq_len or not self._strategy.extend(state, pos):
            return False
        state.length = pos + 1
        return True

    def task_cached(self, task_id: str) -> int:
        state = self._states.get(task_id)
        return state.cached if state is not None else 0

    def task_record_hashes(self, task_id: str, prompt_ids: List[int], start_logical_page: int = 0):
        state = self._states.get(task_id)
        if state is not None:
            self._strategy.record_hashes(state, prompt_ids, start_logical_page)

    @staticmethod
    def task_cacheable_ids(task_id: str, prompt_ids: List[int], output_ids: List[int]) -> List[int]:
        """Tokens whose K/V exist in the pool: the prompt and every output except the last sampled one."""
        return list(prompt_ids) + list(output_ids[:-1])

    def state(self, task_id: str) -> Optional[TaskCacheState]:
        return self._states.get(task_id)

    def bind(self, task_ids: List[str], workspace: InferenceWorkspace, device=None, start_pos: Optional[int] = None,
             start_positions: Optional[List[int]] = None, end_positions: Optional[List[int]] = None) -> KVCache:
        """``end_positions`` (prefill only) stops each request's chunk short of its full length: the keys visible to the
        chunk are ``[0, end)`` and the query rows ``[start, end)``."""
        states = [self._states[t] for t in task_ids]
        rows, lens = [s.req_idx for s in states], [s.length for s in states]
        if end_positions is not None:
            lens = [min(n, e) for n, e in zip(lens, end_positions)]
        sig, prev = tuple(rows), self._bind_state
        decode = start_pos is None and start_positions is None
        steady = (decode and prev is not None and prev.sig == sig and len(prev.seq_lens) == len(lens)
                  and all(c == p + 1 for c, p in zip(lens, prev.seq_lens)))
        self._bind_state = _BindState(sig, list(lens)) if decode else None
        self._bind_was_steady = steady
        return self._pool.bind_tasks(rows, lens, workspace, device=device, start_pos=start_pos, incremental=steady,
                                     start_positions=start_positions)

    @property
    def bind_was_steady(self) -> bool:
        return self._bind_was_steady
