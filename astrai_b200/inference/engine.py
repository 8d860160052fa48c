"""User-facing generation API over the continuous-batching scheduler.

Reference: ``astrai/inference/engine.py:18-242`` (``generate`` for a string, a list, or a streaming generator;
``generate_async``; ``get_stats``; ``shutdown``; 300 s timeout on blocking calls).
"""

from __future__ import annotations

import asyncio
import gc
import threading
from typing import Any, AsyncGenerator, Dict, Generator, List, Optional, Tuple, Union

import torch

from astrai_b200.inference.cache import PagePool
from astrai_b200.inference.scheduler import InferenceScheduler
from astrai_b200.inference.task import STOP


class _PromptStream:
    """Text of one prompt's answer: pieces as they arrive and whether the end marker has been seen."""

    __slots__ = ("pieces", "closed")

    def __init__(self):
        self.pieces: List[str] = []
        self.closed = False


class GenerateResult:
    """Hand-over point between the scheduler thread (producer) and the caller of ``generate`` (consumer).

    Every piece goes into one arrival-ordered inbox (a ``queue.SimpleQueue`` of ``(prompt index, piece)``) that
    streaming consumers drain, and into the per-prompt stream that blocking consumers join at the end.  A
    countdown of open prompts releases ``wait_completion``.  Same calls as ``astrai/inference/engine.py:18-66``:
    ``append``, ``pop_all``, ``wait``, ``wait_completion``, ``get_results``.
    """

    def __init__(self, count: int = 1):
        import queue

        self._empty = queue.Empty
        self._inbox: "queue.SimpleQueue[Tuple[int, Any]]" = queue.SimpleQueue()
        self._held_back: List[Tuple[int, Any]] = []  # items taken by wait() before pop_all() asked for them
        self._streams = [_PromptStream() for _ in range(count)]
        self._open = count
        self._finished = threading.Event()
        self._guard = threading.Lock()
        if count == 0:
            self._finished.set()

    def append(self, token, idx: int = 0):
        stream = self._streams[idx]
        if token is STOP:
            with self._guard:
                if not stream.closed:
                    stream.closed = True
                    self._open -= 1
                    if self._open <= 0:
                        self._finished.set()
        else:
            stream.pieces.append(token)
        self._inbox.put((idx, token))

    def pop_all(self) -> List[Tuple[int, Any]]:
        with self._guard:
            out, self._held_back = self._held_back, []
        while True:
            try:
                out.append(self._inbox.get_nowait())
            except self._empty:
                return out

    def wait(self, timeout: Optional[float] = None) -> bool:
        """Block until something can be popped (True) or ``timeout`` seconds passed (False)."""
        with self._guard:
            if self._held_back:
                return True
        try:
            item = self._inbox.get(timeout=timeout)
        except self._empty:
            return False
        with self._guard:
            self._held_back.append(item)
        return True

    def wait_completion(self, timeout: float = 300.0):
        if not self._finished.wait(timeout=timeout):
            done = sum(s.closed for s in self._streams)
            raise TimeoutError(f"generation still running after {timeout:g} s: {done} of {len(self._streams)} prompts finished")

    def get_results(self) -> List[str]:
        return ["".join(s.pieces) for s in self._streams]


class InferenceEngine:
    def __init__(self, model, tokenizer, max_batch_size: int = 1, max_seq_len: Optional[int] = None,
                 cache: Optional[PagePool] = None, enable_cuda_graph: bool = True, backend=None, **scheduler_kwargs):
        self.model, self.tokenizer = model, tokenizer
        self.scheduler = InferenceScheduler(model=model, tokenizer=tokenizer, max_batch_size=max_batch_size,
                                            max_seq_len=max_seq_len, cache=cache, enable_cuda_graph=enable_cuda_graph,
                                            backend=backend, **scheduler_kwargs)
        # tensor-parallel serving: only the replica's first rank runs the loop in a thread and talks to callers; the
        # other ranks run it in the foreground through follow()
        control = getattr(self.scheduler, "_control", None)
        self.leader = control is None or control.leader
        if self.leader:
            self.scheduler.start()

    def follow(self):
        """Ranks of a tensor-parallel replica other than the first: serve until the first rank shuts the replica down."""
        if self.leader:
            raise RuntimeError("follow() is for the ranks that do not face clients")
        self.scheduler.follow()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.shutdown()
        return False

    def generate(self, prompt: Union[str, List[str]], stream: bool = False, max_tokens: Optional[int] = None,
                 temperature: float = 1.0, top_p: float = 1.0, top_k: int = 50, frequency_penalty: float = 0.0,
                 rep_window: int = 64) -> Union[Generator, str, List[str]]:
        batch = isinstance(prompt, list)
        prompts = prompt if batch else [prompt]
        if max_tokens is not None and max_tokens <= 0:
            if stream:
                return iter(())
            return [""] * len(prompts) if batch else ""
        return self._generate(prompts, batch, stream, max_tokens, temperature, top_p, top_k, frequency_penalty, rep_window)

    def generate_async(self, prompt: str, max_tokens: Optional[int] = None, temperature: float = 1.0, top_p: float = 1.0,
                       top_k: int = 50, frequency_penalty: float = 0.0, rep_window: int = 64,
                       usage: Optional[dict] = None) -> AsyncGenerator[str, None]:
        """Pieces of the answer as an async generator.  Closing it early (``aclose()``, or the consuming coroutine being
        cancelled: a stop sequence matched, the client went away) takes the request out of the scheduler, so that an
        answer nobody reads does not keep a batch slot until ``max_tokens``.  A ``usage`` dict holds, by the time the
        generator ends on its own, ``completion_tokens`` (tokens generated, which the pieces of text undercount) and
        ``finish_reason`` (``stop`` or ``length``)."""
        result, task_ids = self._submit([prompt], max_tokens, temperature, top_p, top_k, frequency_penalty, rep_window,
                                        on_finish=usage.update if usage is not None else None)
        gen = self._stream(result, task_ids, False)

        async def agen():
            loop = asyncio.get_event_loop()
            try:
                while True:
                    piece = await loop.run_in_executor(None, next, gen, None)
                    if piece is None:
                        return
                    yield piece
            finally:
                # not gen.close(): a worker thread may be inside next(gen) right now; ending the streams lets it return
                self._cancel(result, task_ids)

        return agen()

    def _submit(self, prompts, max_tokens, temperature, top_p, top_k, frequency_penalty, rep_window, on_finish=None):
        from astrai_b200.ops.backend import get_backend

        result = GenerateResult(count=len(prompts))
        # a back end chosen by the caller (`with attn_backend(...)`: a per-thread selection) travels with the request to
        # the scheduling thread; None leaves the request on the scheduler's own
        chosen = get_backend(use_default=False)
        extra = {"backend": chosen} if chosen is not None else {}
        if on_finish is not None:
            extra["finish_callback"] = on_finish
        task_ids = [
            self.scheduler.add_task(prompt=p, max_tokens=max_tokens, temperature=temperature, top_p=top_p, top_k=top_k,
                                    frequency_penalty=frequency_penalty, rep_window=rep_window,
                                    stream_callback=lambda tok, i=i: result.append(tok, i), **extra)
            for i, p in enumerate(prompts)
        ]
        return result, task_ids

    def _cancel(self, result: GenerateResult, task_ids: List[str]):
        """Take the requests out (finished ones are gone already: nothing happens) and end their streams."""
        for tid in task_ids:
            self.scheduler.remove_task(tid)
        for i in range(len(task_ids)):
            result.append(STOP, i)

    def _stream(self, result: GenerateResult, task_ids: List[str], batch: bool):
        open_streams = len(task_ids)
        closed = [False] * len(task_ids)
        try:
            while open_streams > 0:
                for idx, tok in result.pop_all():
                    if tok is STOP:
                        if not closed[idx]:
                            closed[idx] = True
                            open_streams -= 1
                    else:
                        yield (idx, tok) if batch else tok
                if open_streams > 0:
                    result.wait(timeout=0.05)
        finally:  # a consumer that stops reading (break, close(), garbage collection) gives the batch slots back
            for tid, done in zip(task_ids, closed):
                if not done:
                    self.scheduler.remove_task(tid)

    def _generate(self, prompts, batch, stream, max_tokens, temperature, top_p, top_k, frequency_penalty, rep_window):
        result, task_ids = self._submit(prompts, max_tokens, temperature, top_p, top_k, frequency_penalty, rep_window)
        if stream:
            return self._stream(result, task_ids, batch)
        try:
            result.wait_completion()
        finally:
            for tid in task_ids:
                self.scheduler.remove_task(tid)
        out = result.get_results()
        return out if batch else out[0]

    def get_stats(self) -> Dict[str, Any]:
        return self.scheduler.get_stats()

    backend_name = property(lambda self: self.scheduler.backend_name)
    cuda_graph_enabled = property(lambda self: self.scheduler.cuda_graph_enabled)

    def shutdown(self):
        self.scheduler.stop()
        if torch.cuda.is_available():
            torch.cuda.empty_cache()
        gc.collect()
