"""Generation requests and the thread-safe queues that hold them.

Rules of the reference (``astrai/inference/task.py:16-290``): a prompt longer than ``max_seq_len`` keeps its LAST
``max_seq_len`` tokens; ``max_tokens = min(requested or inf, max_seq_len - len(prompt))``; a task finishes when it has
produced ``max_tokens`` tokens or its last token is a stop id.
"""

from __future__ import annotations

import threading
import time
import uuid
from collections import deque
from enum import Enum
from typing import Any, Callable, Deque, Dict, List, Optional

STOP = object()


class StreamDecoder:
    """Incremental detokeniser (``tokenizers.decoders.DecodeStream``): returns "" while a multi-byte character is open."""

    __slots__ = ("_stream", "_tok", "_plain")

    def __init__(self, tokenizer):
        from tokenizers.decoders import DecodeStream

        self._tok = getattr(tokenizer, "_tokenizer", None)
        self._plain = tokenizer if self._tok is None else None  # adapters without a `tokenizers` backend: decode per id
        self._stream = DecodeStream(skip_special_tokens=True) if self._tok is not None else None

    def push(self, token_id: int) -> str:
        if self._stream is None:
            return self._plain.decode([token_id]) or ""
        return self._stream.step(self._tok, token_id) or ""


class TaskStatus(Enum):
    PENDING = "pending"
    RUNNING = "running"
    FINISHED = "finished"
    ABORTED = "aborted"


class Task:
    def __init__(self, task_id: str, prompt_ids: List[int], max_tokens: Optional[int] = None, temperature: float = 1.0,
                 top_p: float = 1.0, top_k: int = 50, frequency_penalty: float = 0.0, rep_window: int = 64, backend=None):
        self.task_id, self.prompt_ids, self.max_tokens = task_id, prompt_ids, max_tokens
        self.temperature, self.top_p, self.top_k = temperature, top_p, top_k
        self.frequency_penalty, self.rep_window, self.backend = frequency_penalty, rep_window, backend
        self.status = TaskStatus.PENDING
        self.output_ids: List[int] = []
        self.output_logprobs: List[float] = []
        self.input_tokens = 0
        self.output_tokens = 0
        self._kv_len = 0
        self._decoder: Optional[StreamDecoder] = None
        self.prefill_pos: Optional[int] = None     # chunked prefill: prompt tokens whose K/V are in the cache so far
        self.prefill_start: Optional[int] = None   # first position this task computed itself (after the shared prefix)

    def mark_prefill_done(self):
        self._kv_len = self.input_tokens

    def advance_kv(self):
        self._kv_len += 1

    def decode_new_token(self, tokenizer) -> str:
        if self._decoder is None:
            self._decoder = StreamDecoder(tokenizer)
        return self._decoder.push(self.output_ids[-1])

    @property
    def next_pos(self) -> int:
        return self._kv_len

    @property
    def prefill_done(self) -> bool:
        return self._kv_len >= self.input_tokens > 0

    def is_finished(self, stop_ids) -> bool:
        if self.max_tokens is not None and self.output_tokens >= self.max_tokens:
            return True
        return bool(self.output_ids) and self.output_ids[-1] in stop_ids


class TaskManager:
    def __init__(self, tokenizer, max_batch_size: int = 16, max_seq_len: int = 8192, metrics=None):
        self.tokenizer, self.max_batch_size, self.max_seq_len = tokenizer, max_batch_size, max_seq_len
        self.waiting_queue: Deque[Task] = deque()
        self.active_tasks: List[Task] = []
        self._callbacks: Dict[str, Callable] = {}
        self._finish_callbacks: Dict[str, Callable] = {}
        self._task_event = threading.Event()
        self._lock = threading.Lock()
        self._total_tasks = self._total_tokens = 0
        self._metrics = metrics

    def make_task(self, prompt_ids: List[int], max_tokens: Optional[int], prefix: str = "task", **sampling) -> Optional[Task]:
        if len(prompt_ids) > self.max_seq_len:
            prompt_ids = prompt_ids[-self.max_seq_len:]
        room = self.max_seq_len - len(prompt_ids)
        max_tokens = room if max_tokens is None else min(max_tokens, room)
        return Task(f"{prefix}_{int(time.time())}_{uuid.uuid4().hex[:8]}", list(prompt_ids), max_tokens, **sampling)

    def add_task(self, prompt, max_tokens: Optional[int] = None, temperature: float = 1.0, top_p: float = 1.0,
                 top_k: int = 50, frequency_penalty: float = 0.0, rep_window: int = 64, backend=None,
                 stream_callback: Optional[Callable] = None, finish_callback: Optional[Callable] = None) -> str:
        """``prompt`` is text (tokenised here) or an already tokenised id list.  ``stream_callback`` hears every piece of
        text and then ``STOP``; ``finish_callback`` hears, once and before that ``STOP``, how a request that ran to its end
        ended (see :meth:`report_finish`)."""
        ids = self.tokenizer.encode(prompt) if isinstance(prompt, str) else list(prompt)
        task = self.make_task(ids, max_tokens, temperature=temperature, top_p=top_p, top_k=top_k,
                              frequency_penalty=frequency_penalty, rep_window=rep_window, backend=backend)
        with self._lock:
            self.waiting_queue.append(task)
            self._total_tasks += 1
            if stream_callback:
                self._callbacks[task.task_id] = stream_callback
            if finish_callback:
                self._finish_callbacks[task.task_id] = finish_callback
        if self._metrics is not None:
            self._metrics.register(task.task_id)
        self._task_event.set()
        return task.task_id

    def enqueue(self, task: Task):
        """Append an already built task (tensor-parallel serving: the first rank built it, every rank queues it)."""
        with self._lock:
            self.waiting_queue.append(task)
            self._total_tasks += 1
        if self._metrics is not None:
            self._metrics.register(task.task_id)
        self._task_event.set()

    def register_callback(self, task_id: str, callback: Optional[Callable], finish_callback: Optional[Callable] = None):
        with self._lock:
            if callback is not None:
                self._callbacks[task_id] = callback
            if finish_callback is not None:
                self._finish_callbacks[task_id] = finish_callback

    def report_finish(self, task: Task, stop_ids):
        """Tell the request's ``finish_callback`` the number of tokens generated (text pieces undercount them: a token
        that completes a character only later, or a special token, gives no text) and why generation ended: ``stop`` for
        an end-of-sequence token, ``length`` for a spent token budget or a full context."""
        with self._lock:
            cb = self._finish_callbacks.pop(task.task_id, None)
        if cb:
            ended = bool(task.output_ids) and task.output_ids[-1] in stop_ids
            cb({"completion_tokens": task.output_tokens, "finish_reason": "stop" if ended else "length"})

    def wait_for_wake(self, timeout: float):
        """Sleep until :meth:`wake` (or a new task) or ``timeout`` seconds, whatever the queues hold."""
        self._task_event.clear()
        self._task_event.wait(timeout=timeout)

    def silence(self, task_id: str) -> bool:
        """Stop delivering to the task's callback; True when the task is still queued or running (so that removing it is
        worth a trip through the scheduling loop)."""
        with self._lock:
            self._callbacks.pop(task_id, None)
            self._finish_callbacks.pop(task_id, None)
            return any(t.task_id == task_id for t in self.active_tasks) or any(t.task_id == task_id for t in self.waiting_queue)

    def remove_task(self, task_id: str) -> List[Task]:
        with self._lock:
            gone = [t for t in self.active_tasks if t.task_id == task_id]
            self.waiting_queue = deque(t for t in self.waiting_queue if t.task_id != task_id)
            self.active_tasks = [t for t in self.active_tasks if t.task_id != task_id]
            self._callbacks.pop(task_id, None)
            self._finish_callbacks.pop(task_id, None)
        return gone

    def invoke_callback(self, task_id: str, token):
        cb = self._callbacks.get(task_id)
        if cb:
            cb(token)

    def get_stats(self) -> Dict[str, Any]:
        stats = {"total_tasks": self._total_tasks, "total_tokens": self._total_tokens,
                 "active_tasks": len(self.active_tasks), "waiting_queue": len(self.waiting_queue)}
        if self._metrics is not None:
            stats.update(self._metrics.get_stats())
        return stats

    def remove_finished_tasks(self, stop_ids) -> List[Task]:
        with self._lock:
            done = []
            for t in self.active_tasks:
                if t.status == TaskStatus.ABORTED:
                    done.append(t)
                elif t.is_finished(stop_ids):
                    t.status = TaskStatus.FINISHED
                    done.append(t)
                    self._total_tokens += t.output_tokens
            if self._metrics is not None:
                for t in done:
                    self._metrics.mark_finished(t.task_id, t.input_tokens, t.output_tokens)
            self.active_tasks = [t for t in self.active_tasks if t.status not in (TaskStatus.FINISHED, TaskStatus.ABORTED)]
            for t in done:  # both have heard their last (the loop sends STOP in the iteration before the one that retires)
                self._callbacks.pop(t.task_id, None)
                self._finish_callbacks.pop(t.task_id, None)
            return done

    def pull_candidates(self, n: int) -> List[Task]:
        with self._lock:
            return [self.waiting_queue.popleft() for _ in range(min(n, len(self.waiting_queue)))]

    def activate(self, task: Task):
        task.status = TaskStatus.RUNNING
        with self._lock:
            self.active_tasks.append(task)

    def return_to_waiting(self, tasks: List[Task]):
        with self._lock:
            for t in reversed(tasks):
                self.waiting_queue.appendleft(t)

    def has_work(self) -> bool:
        return bool(self.active_tasks or self.waiting_queue)

    def wait_for_tasks(self, timeout: float = 1.0):
        with self._lock:
            if self.waiting_queue or self.active_tasks:
                return
            self._task_event.clear()
        self._task_event.wait(timeout=timeout)

    def get_active_tasks(self) -> List[Task]:
        with self._lock:
            return list(self.active_tasks)

    def get_waiting_tasks(self) -> List[Task]:
        with self._lock:
            return list(self.waiting_queue)

    def clear_queues(self):
        with self._lock:
            self.waiting_queue.clear()
            self.active_tasks.clear()
            self._callbacks.clear()
            self._finish_callbacks.clear()

    def wake(self):
        self._task_event.set()
