"""Token stores: memory-mapped shards (``bin``) and JSON-lines (``jsonl``).

A store answers two kinds of question (reference ``astrai/dataset/storage.py:67-601``):
* stream access - the data as one long token river cut into windows: ``num_samples = 0 if total <= w else
  (total - 1 - w) // stride + 1``; window ``i`` covers ``[min(i*stride, total-1-w), +w)``;
* record access - the i-th record (bin shards with ``offsets`` in ``meta.json`` - any number of shards, records are
  numbered shard after shard, where the reference gives up on more than one shard - or one JSONL line).
"""

from __future__ import annotations

import bisect
import glob
import json
import logging
from pathlib import Path
from typing import Callable, Dict, List, Optional, Protocol, Tuple, Union, runtime_checkable

import torch
from torch import Tensor

from astrai_b200.factory import BaseFactory
from astrai_b200.serialization import load_bin, load_bin_offsets

logger = logging.getLogger(__name__)
Keys = Union[str, List[str]]


def detect_format(load_path: str) -> str:
    root = Path(load_path)
    if root.is_file():
        if root.suffix.lower() == ".jsonl":
            return "jsonl"
        raise ValueError(f"Unsupported file format: {root.suffix.lower()}")
    if glob.glob(str(root / "**" / "*.bin"), recursive=True) and glob.glob(str(root / "**" / "meta.json"), recursive=True):
        return "bin"
    if glob.glob(str(root / "**" / "*.jsonl"), recursive=True):
        return "jsonl"
    raise FileNotFoundError(f"No supported data files found at {load_path}")


@runtime_checkable
class Streamable(Protocol):
    """A store that serves token ranges of its concatenated keys (``fetch(begin, end, keys)``): windows for ``seq`` /
    ``sft``.  The reference states this as a mixin class (``astrai/dataset/storage.py:314-330``); here it is a
    structural type, so ``isinstance(store, Streamable)`` asks the same question of any store."""

    def fetch(self, begin: int, end: int, keys): ...


@runtime_checkable
class Recordable(Protocol):
    """A store that serves whole records (``fetch_record(index, keys)``): preference pairs, response groups
    (``astrai/dataset/storage.py:361-373``)."""

    def fetch_record(self, index: int, keys): ...


class Store:
    """Holds per-key lists of tensors (segments) and the indices over them."""

    segments_are_records = False

    def __init__(self, window_size: int = 0, stride: Optional[int] = None):
        self._data: Dict[str, list] = {}
        self._cum: Dict[str, List[int]] = {}
        self._offsets: Dict[str, List[Tuple[int, int, int]]] = {}
        self._length = 0
        self._num_records = 0
        self._window_size = int(window_size)
        self._stride = int(stride) if stride else int(window_size)

    def load(self, path: str, **kwargs) -> None:
        raise NotImplementedError

    # -- properties ---------------------------------------------------------------------------------------------
    keys = property(lambda self: list(self._data.keys()))
    window_size = property(lambda self: self._window_size)
    stride = property(lambda self: self._stride)
    token_count = property(lambda self: self._length)
    num_records = property(lambda self: self._num_records)

    def _streaming(self) -> bool:
        return self._window_size > 0 and self._length > 0

    @property
    def num_samples(self) -> int:
        if self._streaming():
            if self._length <= self._window_size:
                return 0
            return (self._length - 1 - self._window_size) // self._stride + 1
        return self._num_records

    def __len__(self) -> int:
        return self.num_samples

    def __getitem__(self, index: int) -> Dict[str, Tensor]:
        n = self.num_samples
        if index < 0:
            index += n
        if not 0 <= index < n:
            raise IndexError(f"Store index out of range: {index}, num_samples={n}")
        if self._streaming():
            b, e = self.sample_window(index)
            return {k: self.fetch(b, e, k) for k in self._stream_keys()}
        return self.fetch_record(index, list(self._data.keys()))

    def sample_window(self, index: int) -> Tuple[int, int]:
        if self._window_size <= 0:
            raise RuntimeError("sample_window() requires window_size > 0 (stream mode)")
        if self._length <= self._window_size:
            raise IndexError(f"Data too short for window: token_count={self._length}, window_size={self._window_size}")
        if not 0 <= index < self.num_samples:
            raise IndexError(f"Sample index out of range: {index}, num_samples={self.num_samples}")
        begin = min(index * self._stride, self._length - 1 - self._window_size)
        return begin, min(begin + self._window_size, self._length - 1)

    def _stream_keys(self) -> List[str]:
        return [k for k, segs in self._data.items() if not (segs and isinstance(segs[0], list))]

    # -- registration ---------------------------------------------------------------------------------------------
    def _normalize(self, raw: Dict[str, list], offsets: Optional[Dict[str, list]] = None):
        lengths = []
        for key, segs in raw.items():
            self._data[key] = segs
            nested = bool(segs) and isinstance(segs[0], list)
            if nested:
                self._cum[key] = []
                continue
            cum, total = [], 0
            for t in segs:
                total += t.shape[0]
                cum.append(total)
            self._cum[key] = cum
            lengths.append(total)
        self._length = min(lengths) if lengths else 0
        # record index per key: (segment, begin, end) of every record.  `offsets[key]` holds one cumulative list per
        # segment (shard) in segment order; a key whose shards do not all carry offsets has no record mode.
        usable: Dict[str, List[Tuple[int, int, int]]] = {}
        for key, per_seg in (offsets or {}).items():
            segs = self._data.get(key, [])
            if per_seg and not isinstance(per_seg[0], (list, tuple)):
                per_seg = [per_seg]
            if len(per_seg) != len(segs):
                logger.warning("Key '%s': %d of %d shards carry record offsets: record mode disabled for it.", key, len(per_seg), len(segs))
                continue
            index = [(si, off[i], off[i + 1]) for si, off in enumerate(per_seg) for i in range(len(off) - 1)]
            if index:
                usable[key] = index
        self._offsets = usable
        if usable:
            self._num_records = min(len(v) for v in usable.values())
        elif self.segments_are_records:
            flat = [len(s) for s in self._data.values() if not (s and isinstance(s[0], list))]
            self._num_records = min(flat) if flat else 0
        else:
            self._num_records = 0

    # -- stream access ----------------------------------------------------------------------------------------------
    def fetch(self, begin: int, end: int, keys: Keys):
        if not self._data:
            raise RuntimeError("Store not loaded")
        if not (0 <= begin < self._length and 0 <= end <= self._length):
            raise ValueError(f"Index out of bounds: begin={begin}, end={end}, length={self._length}")
        if isinstance(keys, str):
            return self._slice(keys, begin, end)
        return {k: self._slice(k, begin, end) for k in keys}

    def _slice(self, key: str, begin: int, end: int) -> Tensor:
        segs, cum = self._data[key], self._cum[key]
        first, last = bisect.bisect_right(cum, begin), bisect.bisect_left(cum, end)
        parts = []
        for i in range(first, last + 1):
            base = cum[i - 1] if i else 0
            parts.append(segs[i][max(begin - base, 0):min(end - base, segs[i].shape[0])])
        return parts[0] if len(parts) == 1 else torch.cat(parts, dim=0)

    # -- record access ------------------------------------------------------------------------------------------------
    def fetch_record(self, index: int, keys: Keys):
        if not self._data and self._num_records == 0:
            raise RuntimeError("Store not loaded")
        if not 0 <= index < self._num_records:
            raise ValueError(f"Record index out of bounds: {index}, num_records={self._num_records}")
        if isinstance(keys, str):
            return self._record(keys, index)
        return {k: self._record(k, index) for k in keys}

    def _record(self, key: str, index: int):
        index_of = self._offsets.get(key)
        if index_of:
            seg, lo, hi = index_of[index]
            return self._data[key][seg][lo:hi]
        return self._data[key][index]


class StoreFactory(BaseFactory["Store"]):
    pass


@StoreFactory.register("bin")
class MmapStore(Store):
    """Every ``meta.json`` below the path is one shard; shards of a key are chained as segments."""

    def load(self, path: str, **kwargs):
        metas = sorted(glob.glob(str(Path(path) / "**" / "meta.json"), recursive=True))
        if not metas:
            raise FileNotFoundError(f"No meta.json found under {path}")
        raw: Dict[str, list] = {}
        offsets: Dict[str, List[List[int]]] = {}
        for meta in metas:
            shard = str(Path(meta).parent)
            for k, segs in load_bin(shard).items():
                raw.setdefault(k, []).extend(segs)
            for k, off in load_bin_offsets(shard).items():
                offsets.setdefault(k, []).append(off)
        self._load_path = path
        self._normalize(raw, offsets=offsets or None)


class JsonlSource:
    """Raw dict records from one ``.jsonl`` file or every ``*.jsonl`` below a directory, in path order (bad lines are
    skipped)."""

    def __init__(self, path: str):
        self.path = Path(path)
        self._records: Optional[List[dict]] = None

    def load(self) -> List[dict]:
        if self._records is None:
            files = [self.path] if self.path.is_file() else sorted(self.path.rglob("*.jsonl"))
            out: List[dict] = []
            for f in files:
                with open(f, "r", encoding="utf-8") as fh:
                    for line in fh:
                        line = line.strip()
                        if not line:
                            continue
                        try:
                            out.append(json.loads(line))
                        except json.JSONDecodeError:
                            logger.warning("Failed to parse JSON line in %s, skipping", f)
            self._records = out
        return self._records


@StoreFactory.register("jsonl")
class JsonlStore(Store):
    """Eager mode tokenises every record at load time with a transform; lazy mode (``processor=``) tokenises per
    ``fetch_record`` call and supports record access only."""

    segments_are_records = True

    def __init__(self, window_size: int = 0, stride: Optional[int] = None):
        super().__init__(window_size, stride)
        self._source: Optional[JsonlSource] = None
        self._processor: Optional[Callable[[dict], Dict[str, Tensor]]] = None
        self._lazy_keys: Optional[List[str]] = None

    def load(self, path: str, transform=None, processor=None, **kwargs):
        self._load_path = path
        self._source = JsonlSource(path)
        records = self._source.load()
        if processor is not None:
            self._processor, self._num_records = processor, len(records)
            return
        if transform is None:
            raise ValueError("JsonlStore eager mode requires transform=. Use DatasetFactory.load() which auto-constructs it.")
        self._normalize(transform.apply(records))

    @property
    def keys(self) -> List[str]:
        if self._processor is None:
            return list(self._data.keys())
        if self._lazy_keys is None and self._num_records > 0:
            self._lazy_keys = list(self._processor(self._source.load()[0]).keys())
        return self._lazy_keys or []

    def fetch_record(self, index: int, keys: Keys):
        if self._processor is None:
            return super().fetch_record(index, keys)
        if not 0 <= index < self._num_records:
            raise ValueError(f"Record index out of bounds: {index}, num_records={self._num_records}")
        data = self._processor(self._source.load()[index])
        return data[keys] if isinstance(keys, str) else {k: data[k] for k in keys}

    def fetch(self, begin: int, end: int, keys: Keys):
        if self._processor is not None:
            raise RuntimeError("JsonlStore in lazy (processor) mode does not support stream fetch(); use fetch_record() instead.")
        return super().fetch(begin, end, keys)

    def __getitem__(self, index: int):
        if self._processor is not None:
            return self.fetch_record(index, self.keys)
        return super().__getitem__(index)
