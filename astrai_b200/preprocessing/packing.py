"""Shard-level packing: truncate, or pack documents into context-sized bins (best-fit decreasing).

Reference: ``astrai/preprocessing/packing.py:14-176``.  A strategy maps ``{key: [per-document lists]}`` to a new dict
with the same keys, applying identical reordering / cutting to every key so per-token alignment is preserved.
"""

from __future__ import annotations

import bisect
from typing import Dict, List

from astrai_b200.factory import BaseFactory

Columns = Dict[str, List[List[int]]]


def _cut(seq: List[int], limit: int, mode: str) -> List[int]:
    if len(seq) <= limit:
        return seq
    return seq[-limit:] if mode == "keep_end" else seq[:limit]


def plan_bfd(sequences: List[List[int]], max_packed_len: int, truncation_mode: str = "keep_start") -> List[List[int]]:
    """Best-fit-decreasing bins of document indices; over-long documents count at ``max_packed_len``.

    Each document goes to the open bin with the least remaining room that still fits it (ties: the earliest bin),
    otherwise it opens a new bin.
    """
    lengths = [min(len(s), max_packed_len) for s in sequences]
    order = sorted(range(len(sequences)), key=lambda i: len(sequences[i]), reverse=True)
    bins: List[List[int]] = []
    room: List[int] = []
    for idx in order:
        need = lengths[idx]
        best, best_room = None, max_packed_len + 1
        for b, r in enumerate(room):
            if need <= r < best_room:
                best, best_room = b, r
        if best is None:
            bins.append([idx])
            room.append(max_packed_len - need)
        else:
            bins[best].append(idx)
            room[best] -= need
    return bins


class PackingStrategy:
    def apply(self, keys: Columns, max_packed_len: int, truncation_mode: str) -> Columns:
        raise NotImplementedError


class PackingStrategyFactory(BaseFactory["PackingStrategy"]):
    pass


@PackingStrategyFactory.register("simple")
class SimplePacking(PackingStrategy):
    """No packing: every document is only truncated to ``max_packed_len``."""

    def apply(self, keys, max_packed_len, truncation_mode):
        return {k: [_cut(v, max_packed_len, truncation_mode) for v in col] for k, col in keys.items()}


@PackingStrategyFactory.register("bfd")
class BFDPacking(PackingStrategy):
    """Documents of one bin are concatenated into one packed sequence (then truncated to the bin size)."""

    def apply(self, keys, max_packed_len, truncation_mode):
        docs = keys.get("sequence", [])
        if not docs:
            return keys
        bins = plan_bfd(docs, max_packed_len, truncation_mode)
        out: Columns = {}
        for k, col in keys.items():
            out[k] = [_cut([tok for i in members for tok in col[i]], max_packed_len, truncation_mode) for members in bins]
        return out


@PackingStrategyFactory.register("bfd_split")
class BFDSplitPacking(BFDPacking):
    """Like ``bfd`` but documents longer than a bin are first cut into bin-sized chunks instead of being truncated."""

    def apply(self, keys, max_packed_len, truncation_mode):
        docs = keys.get("sequence", [])
        if not docs or max_packed_len <= 0:
            return super().apply(keys, max_packed_len, truncation_mode)
        starts = [range(0, len(d), max_packed_len) for d in docs]
        chunked = {k: [v[s:s + max_packed_len] for v, ss in zip(col, starts) for s in ss] for k, col in keys.items()}
        return super().apply(chunked, max_packed_len, truncation_mode)
