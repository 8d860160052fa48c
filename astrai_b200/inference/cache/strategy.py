"""Slot allocation policies: page allocator with ref-counts and LRU reuse, radix prefix index, strategies.

Semantics of ``astrai/inference/cache/strategy.py:24-318``:
* ``Allocator``: free pages first, then the least-recently-released cached page (its index entry is evicted);
  heap of unheld pages + array-threaded ring of retained pages;
* ``RadixCache``: hash-chained index whose links are exact page-sized token tuples; only fully materialised pages
  are shared;
* ``PagedStrategy``: prefix hit -> ``inc_ref`` shared pages, allocate the rest, ``slot = page * page_size + offset``.
"""

from __future__ import annotations

import threading
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
    """Page accounting for the paged KV pool.

    Three disjoint sets: pages in use (reference count > 0), pages nobody holds, and *retained* pages whose
    contents a prefix index still points at.  ``alloc`` prefers an unheld page (lowest index first) and otherwise
    recycles the retained page that was released longest ago, telling ``on_evict`` which one it took.

    Layout: the unheld pages sit in a binary heap; the retained pages form a doubly linked ring threaded through
    two integer arrays (``_fwd`` / ``_back``, slot ``n_pages`` is the ring's sentinel), so taking a page out of the
    middle on a cache hit, refreshing it and popping the oldest are all O(1) with no per-page objects.
    Behaviour follows ``astrai/inference/cache/strategy.py:42-90``.
    """

    _OUT = -1  # link value of a page that is not on the retained ring

    def __init__(self, n_pages: int):
        import heapq

        self.n_pages = n_pages
        self._heap_push, self._heap_pop = heapq.heappush, heapq.heappop
        self._unheld: List[int] = list(range(n_pages))  # already a valid heap
        self._holders = [0] * n_pages
        end = n_pages
        self._fwd = [self._OUT] * n_pages + [end]
        self._back = [self._OUT] * n_pages + [end]
        self._retained = 0
        self.on_evict: Optional[Callable[[int], None]] = None
        self._mutex = threading.Lock()

    # ring helpers (caller holds the mutex)
    def _ring_has(self, page: int) -> bool:
        return self._fwd[page] != self._OUT

    def _ring_unlink(self, page: int):
        nxt, prv = self._fwd[page], self._back[page]
        self._fwd[prv], self._back[nxt] = nxt, prv
        self._fwd[page] = self._back[page] = self._OUT
        self._retained -= 1

    def _ring_push_newest(self, page: int):
        end = self.n_pages
        last = self._back[end]
        self._fwd[last], self._back[page] = page, last
        self._fwd[page], self._back[end] = end, page
        self._retained += 1

    def alloc(self) -> int:
        with self._mutex:
            if self._unheld:
                page = self._heap_pop(self._unheld)
            elif self._retained:
                page = self._fwd[self.n_pages]  # oldest retained page
                self._ring_unlink(page)
                if self.on_evict is not None:
                    self.on_evict(page)
            else:
                return -1
            self._holders[page] = 1
            return page

    def free(self, idx: int, keep_cached: bool = False):
        with self._mutex:
            self._holders[idx] -= 1
            if self._holders[idx] != 0:
                return
            if keep_cached:
                if not self._ring_has(idx):
                    self._ring_push_newest(idx)
            else:
                self._heap_push(self._unheld, idx)

    def inc_ref(self, idx: int):
        with self._mutex:
            self._holders[idx] += 1
            if self._ring_has(idx):
                self._ring_unlink(idx)

    def ref_count(self, idx: int) -> int:
        with self._mutex:
            return self._holders[idx]

    def touch(self, idx: int):
        with self._mutex:
            if self._ring_has(idx):
                self._ring_unlink(idx)
                self._ring_push_newest(idx)

    def available(self) -> int:
        with self._mutex:
            return len(self._unheld) + self._retained


class RadixCache:
    """Prefix index over whole pages of exact token ids.

    A cached prefix is a chain of *links*: link ``n`` is identified by ``(id of link n-1, tokens of page n)``, link
    0 hangs off the root id 0.  All links live in one dictionary keyed by that pair, so a lookup is one hash probe per
    page and there is no tree of node objects; ``_where`` maps a physical page back to its link for eviction.
    Only pages that are completely filled are ever entered.  Dropping a link makes everything chained behind it
    unreachable (those pages stay known to ``has_page`` until they are evicted themselves), which is the sharing
    rule of ``astrai/inference/cache/strategy.py:93-173``.
    """

    ROOT = 0

    def __init__(self, page_size: int):
        self._page_size = page_size
        self._links: Dict[tuple, int] = {}        # (previous link id, page tokens) -> link id
        self._page_of: Dict[int, int] = {}        # link id -> physical page (absent: link exists, contents gone)
        self._key_of: Dict[int, tuple] = {}       # link id -> its key in _links
        self._where: Dict[int, int] = {}          # physical page -> link id
        self._next_id = 1
        self._mutex = threading.Lock()

    def _span(self, token_ids, n: int) -> tuple:
        return tuple(token_ids[n * self._page_size:(n + 1) * self._page_size])

    def lookup(self, token_ids: List[int]) -> List[int]:
        """Physical pages of the longest cached prefix of ``token_ids`` (whole pages only)."""
        with self._mutex:
            pages: List[int] = []
            link = self.ROOT
            for n in range(len(token_ids) // self._page_size):
                link = self._links.get((link, self._span(token_ids, n)))
                page = self._page_of.get(link) if link is not None else None
                if page is None:
                    break
                pages.append(page)
            return pages

    def _forget_page(self, page: int, unlink: bool) -> bool:
        """Returns whether a link left the index (the chain a caller is walking may then be broken)."""
        link = self._where.pop(page, None)
        if link is None:
            return False
        self._page_of.pop(link, None)
        if unlink:
            key = self._key_of.pop(link, None)
            if key is not None and self._links.get(key) == link:
                del self._links[key]
                return True
        return False

    def _descend(self, token_ids, pages: int) -> int:
        """The link reached after ``pages`` whole pages of ``token_ids``, creating the links that are missing."""
        link = self.ROOT
        for n in range(pages):
            key = (link, self._span(token_ids, n))
            nxt = self._links.get(key)
            if nxt is None:
                nxt = self._next_id
                self._next_id += 1
                self._links[key] = nxt
                self._key_of[nxt] = key
            link = nxt
        return link

    def record_chain(self, pages: List[int], token_ids: List[int], start: int = 0):
        """``record(pages[i], token_ids, i)`` for every full page ``i >= start``, in one walk along the chain instead of one
        walk from the root per page (a 4 096-token sequence is 256 pages: 256 steps instead of 33 000)."""
        with self._mutex:
            full = min(len(token_ids) // self._page_size, len(pages))
            if start >= full:
                return
            link = self._descend(token_ids, start)
            for n in range(start, full):
                page = pages[n]
                key = (link, self._span(token_ids, n))
                nxt = self._links.get(key)
                if nxt is not None and self._where.get(page) == nxt:
                    link = nxt  # already entered exactly there: keep the link and whatever is chained behind it
                    continue
                if self._forget_page(page, unlink=True):  # the page was indexed under other tokens; the chain may have lost a link
                    link = self._descend(token_ids, n)
                    key = (link, self._span(token_ids, n))
                    nxt = self._links.get(key)
                if nxt is None:
                    nxt = self._next_id
                    self._next_id += 1
                    self._links[key] = nxt
                    self._key_of[nxt] = key
                old = self._page_of.get(nxt)
                if old is not None and old != page:
                    self._where.pop(old, None)
                self._page_of[nxt] = page
                self._where[page] = nxt
                link = nxt

    def record(self, page_idx: int, token_ids: List[int], logical_page_idx: int):
        """Enter physical page ``page_idx`` as page number ``logical_page_idx`` of the sequence ``token_ids``."""
        with self._mutex:
            if logical_page_idx >= len(token_ids) // self._page_size:
                return  # that page is not full yet
            probe = self.ROOT
            for n in range(logical_page_idx + 1):
                probe = self._links.get((probe, self._span(token_ids, n)))
                if probe is None:
                    break
            if probe is not None and self._where.get(page_idx) == probe:
                return  # already entered exactly there: keep the link (and whatever is chained behind it)
            self._forget_page(page_idx, unlink=True)  # the page may have been indexed under other tokens before
            link = self.ROOT
            for n in range(logical_page_idx + 1):
                key = (link, self._span(token_ids, n))
                nxt = self._links.get(key)
                if nxt is None:
                    nxt = self._next_id
                    self._next_id += 1
                    self._links[key] = nxt
                    self._key_of[nxt] = key
                link = nxt
            old = self._page_of.get(link)
            if old is not None and old != page_idx:
                self._where.pop(old, None)
            self._page_of[link] = page_idx
            self._where[page_idx] = link

    def evict(self, idx: int):
        with self._mutex:
            self._forget_page(idx, unlink=True)

    def has_page(self, idx: int) -> bool:
        with self._mutex:
            return idx in self._where

    def release(self, pages: List[int]) -> None:
        """Kept for interface parity: pages are protected by the allocator's reference counts, not by the index."""


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
        self._prefix.record_chain(state.pages, prompt_ids, start)
