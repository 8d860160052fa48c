"""Lightweight tracing: named ranges that show up in Nsight (NVTX) and in a Chrome-trace file with device times.

Off by default (a disabled range costs one attribute test).  Switch on with ``ASTRAI_B200_TRACE=1`` or
:func:`enable`; the model wraps every decoder layer, the trainer its step phases and the executors their collectives.

* NVTX: each range is pushed / popped on the current thread, so ``nsys`` / ``ncu --nvtx`` group kernels by layer.
* Timeline: with ``record=True`` every range also records a pair of CUDA events (when a GPU is in use) and host
  timestamps into a bounded ring; :func:`export_chrome_trace` writes them as ``chrome://tracing`` JSON, device time
  resolved from the events at export (no synchronisation inside the traced region).

The reference's only tracing is a DEBUG-level CUDA-event timer around prefill / decode forwards
(``astrai/inference/runtime/executor.py:24-45``); that timer lives on as ``inference/runtime/executor.py::timed``.
"""

from __future__ import annotations

import contextlib
import json
import os
import threading
import time
from collections import deque
from typing import Deque, Dict, List, Optional

import torch

_STATE = {"on": os.environ.get("ASTRAI_B200_TRACE", "0") not in ("", "0", "false", "False"), "record": False}
_RING: Deque[Dict] = deque(maxlen=65536)
_LOCK = threading.Lock()


def enable(record: bool = False, capacity: Optional[int] = None):
    """Turn ranges on; ``record`` also keeps them for :func:`export_chrome_trace`."""
    global _RING
    _STATE["on"], _STATE["record"] = True, bool(record)
    if capacity is not None:
        with _LOCK:
            _RING = deque(_RING, maxlen=int(capacity))


def disable():
    _STATE["on"] = _STATE["record"] = False


def enabled() -> bool:
    return _STATE["on"]


def clear():
    with _LOCK:
        _RING.clear()


@contextlib.contextmanager
def range(name: str, device: bool = True):  # noqa: A001 - the NVTX term
    """``with trace.range("layer3"):`` - a no-op unless tracing is on."""
    if not _STATE["on"]:
        yield
        return
    cuda = device and torch.cuda.is_available() and torch.cuda.is_initialized()
    if cuda:
        torch.cuda.nvtx.range_push(name)
    rec = None
    if _STATE["record"]:
        rec = {"name": name, "tid": threading.get_ident(), "t0": time.perf_counter(), "t1": None, "e0": None, "e1": None}
        if cuda:
            rec["e0"] = torch.cuda.Event(enable_timing=True)
            rec["e1"] = torch.cuda.Event(enable_timing=True)
            rec["e0"].record()
    try:
        yield
    finally:
        if rec is not None:
            if rec["e1"] is not None:
                rec["e1"].record()
            rec["t1"] = time.perf_counter()
            with _LOCK:
                _RING.append(rec)
        if cuda:
            torch.cuda.nvtx.range_pop()


def mark(name: str):
    """An instantaneous marker (NVTX mark + zero-length timeline entry)."""
    if not _STATE["on"]:
        return
    if torch.cuda.is_available() and torch.cuda.is_initialized():
        torch.cuda.nvtx.mark(name)
    if _STATE["record"]:
        now = time.perf_counter()
        with _LOCK:
            _RING.append({"name": name, "tid": threading.get_ident(), "t0": now, "t1": now, "e0": None, "e1": None})


def events() -> List[Dict]:
    """Recorded ranges as dicts: name, host start / duration in ms, device duration in ms (None without a GPU)."""
    with _LOCK:
        recs = list(_RING)
    if any(r["e1"] is not None for r in recs):
        torch.cuda.synchronize()
    out = []
    for r in recs:
        dev_ms = None
        if r["e0"] is not None and r["e1"] is not None:
            try:
                dev_ms = r["e0"].elapsed_time(r["e1"])
            except RuntimeError:
                dev_ms = None
        out.append({"name": r["name"], "tid": r["tid"], "host_start_ms": r["t0"] * 1e3,
                    "host_ms": (r["t1"] - r["t0"]) * 1e3, "device_ms": dev_ms})
    return out


def export_chrome_trace(path: str, rank: Optional[int] = None) -> int:
    """Write the recorded ranges as Chrome-trace JSON (one row per thread; device durations on a second process row).
    Returns the number of ranges written."""
    evs = events()
    pid = int(os.environ.get("RANK", "0")) if rank is None else rank
    rows = []
    for e in evs:
        rows.append({"name": e["name"], "ph": "X", "pid": pid, "tid": e["tid"], "ts": e["host_start_ms"] * 1e3,
                     "dur": max(e["host_ms"], 0.0) * 1e3, "args": {"device_ms": e["device_ms"]}})
        if e["device_ms"] is not None:
            rows.append({"name": e["name"], "ph": "X", "pid": f"{pid}-device", "tid": e["tid"], "ts": e["host_start_ms"] * 1e3,
                         "dur": e["device_ms"] * 1e3})
    with open(path, "w") as fh:
        json.dump({"traceEvents": rows, "displayTimeUnit": "ms"}, fh)
    return len(evs)
