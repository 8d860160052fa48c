"""Per-request serving metrics: queue wait, TTFT, prefill / decode rates, end-to-end latency, rolling averages.

Field names of ``GET /stats`` follow ``astrai/inference/metrics.py:10-201``; percentile summaries are an addition.
"""

from __future__ import annotations

import time
from collections import deque
from contextlib import contextmanager
from dataclasses import dataclass
from typing import Any, Deque, Dict, List, Optional


def _r(v: Optional[float]) -> Optional[float]:
    return None if v is None else round(v, 2)


@dataclass
class TaskTiming:
    task_id: str
    arrival_time: float
    prefill_start_time: Optional[float] = None
    first_token_time: Optional[float] = None
    finish_time: Optional[float] = None
    input_tokens: int = 0
    output_tokens: int = 0
    _decode_steps: int = 0
    _decode_total_s: float = 0.0

    @staticmethod
    def _span_ms(a: Optional[float], b: Optional[float]) -> Optional[float]:
        return None if a is None or b is None else (b - a) * 1000

    queue_wait_ms = property(lambda s: s._span_ms(s.arrival_time, s.prefill_start_time))
    ttft_ms = property(lambda s: s._span_ms(s.arrival_time, s.first_token_time))
    e2e_latency_ms = property(lambda s: s._span_ms(s.arrival_time, s.finish_time))

    @property
    def prefill_tps(self):
        d = self._span_ms(self.prefill_start_time, self.first_token_time)
        return self.input_tokens / (d / 1000) if d and self.input_tokens > 0 else None

    @property
    def decode_tps(self):
        d = self._span_ms(self.first_token_time, self.finish_time)
        return (self.output_tokens - 1) / (d / 1000) if d and self.output_tokens > 1 else None

    @property
    def decode_avg_ms(self):
        return self._decode_total_s / self._decode_steps * 1000 if self._decode_steps and self._decode_total_s > 0 else None

    @property
    def total_tps(self):
        d = self.e2e_latency_ms
        n = self.input_tokens + self.output_tokens
        return n / (d / 1000) if d and n > 0 else None

    def to_dict(self) -> Dict[str, Any]:
        return {"task_id": self.task_id, "input_tokens": self.input_tokens, "output_tokens": self.output_tokens,
                "queue_wait_ms": _r(self.queue_wait_ms), "ttft_ms": _r(self.ttft_ms), "prefill_tps": _r(self.prefill_tps),
                "decode_tps": _r(self.decode_tps), "decode_avg_ms": _r(self.decode_avg_ms), "total_tps": _r(self.total_tps),
                "e2e_latency_ms": _r(self.e2e_latency_ms)}


class MetricsCollector:
    def __init__(self, max_recent: int = 128):
        self._timings: Dict[str, TaskTiming] = {}
        self._completed: Deque[TaskTiming] = deque(maxlen=max_recent)
        self._sums = {"ttft": [0.0, 0], "decode_tps": [0.0, 0], "e2e": [0.0, 0]}
        self.history: List[TaskTiming] = []  # every finished task (benchmarks read percentiles from here)
        self.keep_history = False

    def register(self, task_id: str, arrival_time: Optional[float] = None):
        self._timings[task_id] = TaskTiming(task_id, arrival_time if arrival_time is not None else time.time())

    def mark_finished(self, task_id: str, input_tokens: int, output_tokens: int):
        t = self._timings.pop(task_id, None)
        if t is None:
            return
        t.finish_time, t.input_tokens, t.output_tokens = time.time(), input_tokens, output_tokens
        self._completed.append(t)
        if self.keep_history:
            self.history.append(t)
        for key, val in (("ttft", t.ttft_ms), ("decode_tps", t.decode_tps), ("e2e", t.e2e_latency_ms)):
            if val is not None:
                self._sums[key][0] += val
                self._sums[key][1] += 1

    @contextmanager
    def record(self, task_ids: List[str], phase: str):
        tic = time.time()
        yield
        toc = time.time()
        for tid in task_ids:
            t = self._timings.get(tid)
            if t is None:
                continue
            if phase == "prefill":
                if t.prefill_start_time is None:
                    t.prefill_start_time = tic
                t.first_token_time = toc
            elif phase == "decode":
                t._decode_steps += 1
                t._decode_total_s += toc - tic

    def get_stats(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {}
        for key, name in (("ttft", "avg_ttft_ms"), ("decode_tps", "avg_decode_tps"), ("e2e", "avg_e2e_latency_ms")):
            total, n = self._sums[key]
            if n:
                out[name] = round(total / n, 2)
        if self._completed:
            out["recent_tasks"] = [t.to_dict() for t in self._completed]
        return out
