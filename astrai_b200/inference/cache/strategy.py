"""Slot allocation policies: page allocator with ref-counts and LRU reuse, radix prefix index, strategies.

Semantics of ``astrai/inference/cache/strategy.py:24-318``:
* ``Allocator``: free pages first, then the least-recently-released cached page (its index entry is evicted);
* ``RadixCache``: trie whose edges are exact page-sized token tuples; only fully materialised pages are shared;
* ``PagedStrategy``: prefix hit -> ``inc_ref`` shared pages, allocate the rest, ``slot = page * page_size + offset``.
"""

from __future__ import annotations

import threading
from collections import OrderedDict
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional

import torch

from astrai_b200.inference.cache.buffer import ReqToTokenPool


@dataclass
class TaskCacheState:
    req_idx: int
    length: int = 0
    cached: int = 0
    pages: List[int] = field(default_factory=list)


class Allocator:
    def __init__(self, n_pages: int):
        self.n_pages = n_pages
        self._free: List[int] = list(range(n_pages - 1, -1, -1))  # pop() hands out the lowest index first
        self._refs = [0] * n_pages
        self._lru: "OrderedDict[int, None]" = OrderedDict()
        self.on_evict: Optional[Callable[[int], None]] = None
        self._lock = threading.Lock()

    def alloc(self) -> int:
        with self._lock:
            if self._free:
                idx = self._free.pop()
            elif self._lru:
                idx, _ = self._lru.popitem(last=False)
                if self.on_evict:
                    self.on_evict(idx)
            else:
                return -1
            self._refs[idx] = 1
            return idx

    def free(self, idx: int, keep_cached: bool = False):
        with self._lock:
            self._refs[idx] -= 1
            if self._refs[idx] == 0:
                if keep_cached:
                    self._lru[idx] = None
                else:
                    self._free.append(idx)

    def inc_ref(self, idx: int):
        with self._lock:
            self._refs[idx] += 1
            self._lru.pop(idx, None)

    def ref_count(self, idx: int) -> int:
        with self._lock:
            return self._refs[idx]

    def touch(self, idx: int):
        with self._lock:
            if idx in self._lru:
                self._lru.move_to_end(idx)

    def available(self) -> int:
        with self._lock:
            return len(self._free) + len(self._lru)


class RadixNode:
    __slots__ = ("parent", "children", "page_idx", "tokens", "lock_ref")

    def __init__(self, parent=None, tokens=(), page_idx=None):
        self.parent, self.tokens, self.page_idx = parent, tuple(tokens), page_idx
        self.children: Dict[tuple, "RadixNode"] = {}
        self.lock_ref = 0


class RadixCache:
    def __init__(self, page_size: int):
        self._page_size = page_size
        self._root = RadixNode()
        self._page_to_node: Dict[int, RadixNode] = {}
        self._lock = threading.Lock()

    def _page_tokens(self, token_ids, i):
        return tuple(token_ids[i * self._page_size:(i + 1) * self._page_size])

    def lookup(self, token_ids: List[int]) -> List[int]:
        with self._lock:
            hits, node = [], self._root
            for i in range(len(token_ids) // self._page_size):
                node = node.children.get(self._page_tokens(token_ids, i))
                if node is None or node.page_idx is None:
                    break
                hits.append(node.page_idx)
            return hits

    def record(self, page_idx: int, token_ids: List[int], logical_page_idx: int):
        with self._lock:
            if logical_page_idx >= len(token_ids) // self._page_size:
                return
            stale = self._page_to_node.pop(page_idx, None)
            if stale is not None and stale.parent is not None:
                stale.parent.children.pop(stale.tokens, None)
            node = self._root
            for i in range(logical_page_idx + 1):
                key = self._page_tokens(token_ids, i)
                nxt = node.children.get(key)
                if nxt is None:
                    nxt = node.children[key] = RadixNode(node, key)
                node = nxt
            if node.page_idx is not None and node.page_idx != page_idx:
                self._page_to_node.pop(node.page_idx, None)
            node.page_idx = page_idx
            self._page_to_node[page_idx] = node

    def evict(self, idx: int):
        with self._lock:
            node = self._page_to_node.pop(idx, None)
            if node is None:
                return
            node.page_idx = None
            if node.parent is not None:
                node.parent.children.pop(node.tokens, None)

    def has_page(self, idx: int) -> bool:
        with self._lock:
            return idx in self._page_to_node

    def release(self, pages: List[int]) -> None:
        with self._lock:
            for p in pages:
                node = self._page_to_node.get(p)
                if node is not None and node.lock_ref:
                    node.lock_ref -= 1


class AllocationStrategy:
    def alloc(self, state: TaskCacheState, prompt_ids: List[int]) -> bool:
        raise NotImplementedError

    def free(self, state: TaskCacheState) -> None:
        raise NotImplementedError

    def extend(self, state: TaskCacheState, pos: int) -> bool:
        raise NotImplementedError

    def write_indices(self, state: TaskCacheState, prompt_ids: List[int]) -> None:
        raise NotImplementedError

    def record_hashes(self, state: TaskCacheState, prompt_ids: List[int], start: int) -> None:
        raise NotImplementedError


class ContiguousStrategy(AllocationStrategy):
    """Each request row owns a fixed contiguous slot range written once at pool construction."""

    def alloc(self, state, prompt_ids):
        return True

    def free(self, state):
        pass

    def extend(self, state, pos):
        return True

    def write_indices(self, state, prompt_ids):
        pass

    def record_hashes(self, state, prompt_ids, start):
        pass


class PagedStrategy(AllocationStrategy):
    def __init__(self, alloc: Allocator, prefix: Optional[RadixCache], page_size: int, req_pool: ReqToTokenPool, device):
        self._alloc, self._prefix, self._page_size, self._req_pool, self._device = alloc, prefix, page_size, req_pool, device
        self._offsets = torch.arange(page_size, dtype=torch.int32)

    def _slots(self, pages: List[int]) -> torch.Tensor:
        base = torch.tensor(pages, dtype=torch.int32) * self._page_size
        return (base[:, None] + self._offsets[None, :]).reshape(-1)

    def alloc(self, state, prompt_ids):
        if self._prefix is not None:
            hits = self._prefix.lookup(prompt_ids)
            for p in hits:
                self._alloc.inc_ref(p)
            state.pages, state.cached = list(hits), len(hits) * self._page_size
        remaining = len(prompt_ids) - state.cached
        for _ in range(max(0, -(-remaining // self._page_size))):
            p = self._alloc.alloc()
            if p < 0:
                return False
            state.pages.append(p)
        return True

    def free(self, state):
        for p in state.pages:
            keep = self._prefix is not None and self._prefix.has_page(p)
            self._alloc.free(p, keep_cached=keep)
            if self._prefix is not None and not keep:
                self._prefix.evict(p)
        state.pages = []

    def extend(self, state, pos):
        page = pos // self._page_size
        if page >= len(state.pages):
            p = self._alloc.alloc()
            if p < 0:
                return False
            state.pages.append(p)
            begin = page * self._page_size
            room = min(self._page_size, self._req_pool.max_context_len - begin)
            self._req_pool.write_row(state.req_idx, begin, self._slots([p])[:room])  # the whole page in one copy
        return True

    def write_indices(self, state, prompt_ids):
        if not state.pages:
            return
        slots = self._slots(state.pages)[: self._req_pool.max_context_len]
        self._req_pool.write_row(state.req_idx, 0, slots)

    def record_hashes(self, state, prompt_ids, start):
        if self._prefix is None:
            return
        for i in range(start, min(len(prompt_ids) // self._page_size, len(state.pages))):
            self._prefix.record(state.pages[i], prompt_ids, i)
