"""Continuous-batching scheduler: cleanup -> refill -> prefill new requests -> decode the rest, on a daemon thread.

Loop structure, radix-cache bookkeeping and the synchronous ``run_batch`` path follow
``astrai/inference/scheduler.py:25-400``.  Differences: the KV pool is paged (16-token pages) with the radix prefix
index by default; all requests that need prefill in a step run in ONE packed forward regardless of their lengths,
bounded by ``max_prefill_tokens``; requests that cannot be given cache pages wait instead of failing.
"""

from __future__ import annotations

import contextlib
import logging
import threading
import uuid
from typing import Any, Dict, List, Optional, Tuple

import torch

from astrai_b200.inference.cache import PagePool, TaskCacheManager
from astrai_b200.inference.metrics import MetricsCollector
from astrai_b200.inference.runtime.executor import Executor
from astrai_b200.inference.task import STOP, Task, TaskManager, TaskStatus
from astrai_b200.ops import backend as attn_backends

logger = logging.getLogger(__name__)


class InferenceScheduler:
    def __init__(self, model, tokenizer, max_batch_size: int = 16, max_seq_len: Optional[int] = None, device=None,
                 dtype=None, cache: Optional[PagePool] = None, enable_cuda_graph: bool = True, backend=None,
                 page_size: int = 16, kv_cache_tokens: Optional[int] = None, paged: bool = True,
                 max_prefill_tokens: int = 8192, chunked_prefill: bool = False, prefill_defer_steps: int = 8,
                 prefill_defer_min_batch: int = 32, prefill_defer_tokens: int = 2048, tp_group=None, tp_size: int = 1):
        """``tp_size > 1`` (or a ``tp_group``): tensor-parallel serving - the model is cut over the ranks of the group,
        every rank runs this scheduler in lockstep and the first rank alone talks to clients
        (:mod:`astrai_b200.parallel.tp_inference`; the other ranks call :meth:`follow`)."""
        self._control = None
        if tp_group is not None or tp_size > 1:
            from astrai_b200.parallel.tp_inference import ReplicatedControl, shard_for_inference_

            self._control = ReplicatedControl(tp_group)
            if getattr(model, "tp_size", 1) == 1:
                shard_for_inference_(model, self._control.world, self._control.rank, tp_group)
        cfg = getattr(model, "local_config", None) or model.config
        if max_seq_len is None:
            max_seq_len = cfg.max_position_embeddings
        if max_seq_len is None:
            raise ValueError("max_seq_len must be provided either as argument or in model config (config.max_position_embeddings)")
        self.max_seq_len = max_seq_len
        p = next(model.parameters())
        self.device = torch.device(device) if device is not None else p.device
        self.dtype = dtype or p.dtype
        self._cache = cache if cache is not None else PagePool.for_model(
            cfg, max_batch_size, max_seq_len, self.device, self.dtype, page_size=page_size, n_tokens=kv_cache_tokens, paged=paged)
        self._metrics = MetricsCollector()
        self._task_cache = TaskCacheManager(self._cache)
        self._task_mgr = TaskManager(tokenizer, max_batch_size, max_seq_len, metrics=self._metrics)
        # `backend`: the attention back end of this scheduler's forwards (name or ATTN_BACKEND; None = the process default).
        # Context selections are per thread, so the loop thread enters it itself; decode graphs are captured under it.
        self._backend = attn_backends.resolve(backend) if backend is not None else None
        with self._backend_context():
            self._executor = Executor(model, self._cache, self._task_cache, self.device, self.dtype, enable_cuda_graph,
                                      max_prefill_tokens=max_prefill_tokens, control=self._control)
            active = attn_backends.get_backend(self.device.type)
            self._backend_name = active.value if isinstance(active, attn_backends.ATTN_BACKEND) else type(active).__name__
        self._staged: List[dict] = []      # tensor-parallel serving, first rank: requests not yet shared with the others
        self._cancelled: List[str] = []
        self._stage_lock = threading.Lock()
        self._batch_serial = 0
        self.max_prefill_tokens = max_prefill_tokens
        # chunked prefill: at most max_prefill_tokens prompt tokens per step over all requests; a long prompt takes
        # several steps and the running requests keep decoding in between (the reference never mixes the two)
        self.chunked_prefill = chunked_prefill
        # Admission of new prompts under load: a prefill forward is hundreds of eager launches whatever its size, so with
        # at least `prefill_defer_min_batch` requests decoding, newly arrived prompts wait until `prefill_defer_tokens`
        # prompt tokens are pending or `prefill_defer_steps` decode steps have passed, and are then prefilled together
        # (0 steps = never wait).  With a small decode batch a new prompt is prefilled at once.
        self.prefill_defer_steps, self.prefill_defer_min_batch = int(prefill_defer_steps), int(prefill_defer_min_batch)
        self.prefill_defer_tokens = int(prefill_defer_tokens)
        self._steps_since_prefill = 0
        self._stop_event = threading.Event()
        self._loop_thread: Optional[threading.Thread] = None

    def _backend_context(self, backend=None):
        chosen = backend if backend is not None else self._backend
        return attn_backends.attn_backend(chosen) if chosen is not None else contextlib.nullcontext()

    # -- public surface -----------------------------------------------------------------------------------------------------
    def add_task(self, prompt, **kwargs) -> str:
        if self._control is None:
            return self._task_mgr.add_task(prompt, **kwargs)
        if not self._control.leader:
            raise RuntimeError("requests enter a tensor-parallel replica through its first rank")
        # staged: the request joins the queue of every rank at the start of the next loop iteration, in arrival order
        callback, on_finish = kwargs.pop("stream_callback", None), kwargs.pop("finish_callback", None)
        backend = kwargs.pop("backend", None)
        ids = self._task_mgr.tokenizer.encode(prompt) if isinstance(prompt, str) else list(prompt)
        task = self._task_mgr.make_task(ids, kwargs.pop("max_tokens", None), **kwargs)
        spec = {"task_id": task.task_id, "prompt_ids": task.prompt_ids, "max_tokens": task.max_tokens, "temperature": task.temperature,
                "top_p": task.top_p, "top_k": task.top_k, "frequency_penalty": task.frequency_penalty, "rep_window": task.rep_window}
        with self._stage_lock:
            self._staged.append(spec)
            if callback is not None or on_finish is not None:
                self._task_mgr.register_callback(task.task_id, callback, on_finish)
        self._task_mgr.wake()
        return task.task_id

    def remove_task(self, task_id: str):
        """Take a request out, wherever it is.  Its callback hears nothing more from now on; while the scheduling loop runs,
        the request itself leaves at the top of the loop's next iteration, on the loop's thread (its cache pages may be in
        use by the step in flight, and the page tables have one writer)."""
        if self._control is not None:
            with self._stage_lock:
                self._cancelled.append(task_id)
            return
        running = self._loop_thread is not None and self._loop_thread.is_alive() and threading.current_thread() is not self._loop_thread
        if not running:
            self._drop(task_id)
        elif self._task_mgr.silence(task_id):
            with self._stage_lock:
                self._cancelled.append(task_id)
            self._task_mgr.wake()

    def _drop(self, task_id: str):
        for task in self._task_mgr.remove_task(task_id):
            self._task_cache.task_free(task.task_id)

    def _apply_cancellations(self):
        if not self._cancelled:
            return
        with self._stage_lock:
            gone, self._cancelled = self._cancelled, []
        for task_id in gone:
            self._drop(task_id)

    def _share_requests(self) -> bool:
        """Tensor-parallel serving: bring the queues of every rank up to date with what reached the first rank since the
        last iteration.  Returns False when the replica is to stop."""
        payload = None
        if self._control.leader:
            with self._stage_lock:
                payload = {"new": self._staged, "cancelled": self._cancelled, "stop": self._stop_event.is_set()}
                self._staged, self._cancelled = [], []
        payload = self._control.share(payload)
        for spec in payload["new"]:
            self._task_mgr.enqueue(Task(spec["task_id"], list(spec["prompt_ids"]), spec["max_tokens"], spec["temperature"], spec["top_p"],
                                        spec["top_k"], spec["frequency_penalty"], spec["rep_window"]))
        for task_id in payload["cancelled"]:
            self._drop(task_id)
        return not payload["stop"]

    def follow(self):
        """Run the scheduling loop on the calling thread until the first rank stops the replica (ranks other than the first)."""
        self._stop_event.clear()
        self._run_generation_loop()
        self._abort_and_clear(free_waiting=True)

    def get_stats(self) -> Dict[str, Any]:
        return self._task_mgr.get_stats()

    backend_name = property(lambda self: self._backend_name)
    cuda_graph_enabled = property(lambda self: self._executor.cuda_graph_enabled)
    metrics = property(lambda self: self._metrics)
    cache = property(lambda self: self._cache)

    # -- one scheduling step -------------------------------------------------------------------------------------------------
    def _prefill_batches(self, tasks: List[Task]) -> List[List[Task]]:
        """Greedy split of the prefill set so that no packed forward exceeds the token budget."""
        batches, cur, used = [], [], 0
        for t in tasks:
            need = len(t.prompt_ids) - min(self._task_cache.task_cached(t.task_id), len(t.prompt_ids) - 1)
            if cur and used + need > self.max_prefill_tokens:
                batches.append(cur)
                cur, used = [], 0
            cur.append(t)
            used += need
        if cur:
            batches.append(cur)
        return batches

    def _prefill_chunk(self, tasks: List[Task]) -> Tuple[List[Task], Dict[str, int]]:
        """Chunked prefill: the requests (in arrival order) and chunk ends that fit this step's token budget."""
        group, ends, left = [], {}, self.max_prefill_tokens
        for t in tasks:
            if left <= 0:
                break
            n = len(t.prompt_ids)
            start = t.prefill_pos if t.prefill_pos is not None else min(self._task_cache.task_cached(t.task_id), n - 1)
            take = min(n - start, left)
            group.append(t)
            ends[t.task_id] = start + take
            left -= take
        return group, ends

    def _defer_prefill(self, fresh: List[Task], n_decoding: int) -> bool:
        if not fresh or self.prefill_defer_steps <= 0 or n_decoding < self.prefill_defer_min_batch:
            return False
        if self._steps_since_prefill >= self.prefill_defer_steps:
            return False
        pending = 0
        for t in fresh:
            done = t.prefill_pos if t.prefill_pos is not None else min(self._task_cache.task_cached(t.task_id), len(t.prompt_ids) - 1)
            pending += len(t.prompt_ids) - done
        return pending < self.prefill_defer_tokens

    def _step(self, tasks: List[Task], return_logprobs: bool = False, one_backend: bool = False) -> Tuple[List[Task], List[Task]]:
        """Advance every task by one token.  Returns (tasks that produced a token, tasks aborted for lack of room).

        The decode forward of the requests that are past their prompt is launched first (one graph replay) and the
        prefill forward of the new prompts is issued while it runs; the sampled tokens of both are read back afterwards,
        so the host time of the prefill launches overlaps the decode step on the GPU.

        Requests that were submitted under an attention back end of their own (``Task.backend``, captured from the
        submitting thread's ``attn_backend(...)`` context) are stepped group by group under that back end, as the
        reference does (``astrai/inference/scheduler.py:125-214``)."""
        if not one_backend and any(t.backend is not None for t in tasks):
            groups: Dict[Any, List[Task]] = {}
            for t in tasks:
                groups.setdefault(t.backend, []).append(t)
            stepped, aborted = [], []
            for backend, group in groups.items():
                with self._backend_context(backend):
                    done, gone = self._step(group, return_logprobs, one_backend=True)
                stepped += done
                aborted += gone
            return stepped, aborted
        fresh = [t for t in tasks if not t.prefill_done and t.prompt_ids]
        decode, aborted = [], []
        for t in tasks:
            if not t.prefill_done:
                continue
            if self._task_cache.task_extend(t.task_id, t.next_pos):
                decode.append(t)
            else:
                t.status = TaskStatus.ABORTED
                aborted.append(t)
        if self._defer_prefill(fresh, len(decode)):
            plan = []
            self._steps_since_prefill += 1
        elif self.chunked_prefill:
            group, ends = self._prefill_chunk(fresh)
            plan = [(group, ends)] if group else []
        else:
            plan = [(g, None) for g in self._prefill_batches(fresh)]
        if plan:
            self._steps_since_prefill = 0
        first: List[Task] = []
        with self._metrics.record([t.task_id for t in decode], "decode"):
            read_decode = self._executor.execute_decode(decode, return_logprobs=return_logprobs, wait=False) if decode else None
            for group, ends in plan:
                for t in group:
                    t.input_tokens = len(t.prompt_ids)
                with self._metrics.record([t.task_id for t in group], "prefill"):
                    ordered, read = self._executor.execute_prefill(group, return_logprobs=return_logprobs, end_positions=ends,
                                                                   wait=False)
                    outs = read()
                for t, o in zip(ordered, outs):
                    t.output_ids.append(o[0] if return_logprobs else o)
                    t.output_tokens += 1
                    t.mark_prefill_done()
                    first.append(t)
                    # pages fully covered by the prompt become shareable from the first recomputed page on
                    self._task_cache.task_record_hashes(t.task_id, t.prompt_ids, (t.prefill_start or 0) // self._cache.page_size)
            if read_decode is not None:
                for t, o in zip(decode, read_decode()):
                    t.output_ids.append(o[0] if return_logprobs else o)
                    t.output_tokens += 1
                    t.advance_kv()
        return first + decode, aborted

    def _retire(self, stop_ids):
        for task in self._task_mgr.remove_finished_tasks(stop_ids):
            if task.status == TaskStatus.FINISHED:
                ids = self._task_cache.task_cacheable_ids(task.task_id, task.prompt_ids, task.output_ids)
                self._task_cache.task_record_hashes(task.task_id, ids)
            self._task_cache.task_free(task.task_id)

    def _refill(self):
        room = self._task_mgr.max_batch_size - len(self._task_mgr.get_active_tasks())
        if room <= 0:
            return
        rejected = []
        for task in self._task_mgr.pull_candidates(room):
            if self._task_cache.task_alloc(task.task_id, task.prompt_ids):
                self._task_mgr.activate(task)
            else:
                rejected.append(task)
        if rejected:
            self._task_mgr.return_to_waiting(rejected)

    def _run_generation_loop(self):
        with self._backend_context():
            self._generation_loop()

    def _generation_loop(self):
        tok = self._task_mgr.tokenizer
        stop_ids = set(tok.stop_ids)
        try:
            while True:
                if self._control is not None:
                    if not self._share_requests():
                        break
                elif self._stop_event.is_set():
                    break
                self._retire(stop_ids)  # first: a request that has just finished is counted and its pages are indexed
                if self._control is None:
                    self._apply_cancellations()
                self._refill()
                active = self._task_mgr.get_active_tasks()
                if not active:
                    if self._control is not None:
                        # only the first rank idles (briefly, until a request is staged); the others wait in the next broadcast
                        if self._control.leader and not self._staged and not self._stop_event.is_set():
                            self._task_mgr.wait_for_wake(timeout=0.02)
                    elif not self._task_mgr.has_work():
                        self._task_mgr.wait_for_tasks(timeout=1.0)
                    else:
                        self._stop_event.wait(0.001)  # waiting requests do not fit yet
                    continue
                decoded, aborted = self._step(active)
                for t in aborted:
                    self._task_mgr.invoke_callback(t.task_id, STOP)
                for t in decoded:
                    text = t.decode_new_token(tok)
                    if text:
                        self._task_mgr.invoke_callback(t.task_id, text)
                    if t.is_finished(stop_ids):
                        self._task_mgr.report_finish(t, stop_ids)
                        self._task_mgr.invoke_callback(t.task_id, STOP)
        except Exception as exc:  # noqa: BLE001 - every waiter must be released
            self._stop_event.set()
            logger.error("Scheduler loop crashed: %s", exc, exc_info=True)
            self._abort_and_clear(free_waiting=False)

    def start(self):
        if self._loop_thread is not None and self._loop_thread.is_alive():
            return
        self._stop_event.clear()
        self._loop_thread = threading.Thread(target=self._run_generation_loop, daemon=True, name="astrai-b200-scheduler")
        self._loop_thread.start()

    def stop(self):
        self._stop_event.set()
        self._task_mgr.wake()
        if self._loop_thread is not None:
            self._loop_thread.join(timeout=5.0)
        self._loop_thread = None
        self._abort_and_clear(free_waiting=True)

    def _abort_and_clear(self, free_waiting: bool):
        for t in self._task_mgr.get_active_tasks():
            self._task_mgr.invoke_callback(t.task_id, STOP)
            self._task_cache.task_free(t.task_id)
        for t in self._task_mgr.get_waiting_tasks():
            self._task_mgr.invoke_callback(t.task_id, STOP)
            if free_waiting:
                self._task_cache.task_free(t.task_id)
        self._task_mgr.clear_queues()

    # -- synchronous path (RL rollout) -------------------------------------------------------------------------------------------
    def run_batch(self, prompt_ids_list: List[List[int]], *, max_tokens: Optional[int] = None, temperature: float = 1.0,
                  top_p: float = 1.0, top_k: int = 50, frequency_penalty: float = 0.0, rep_window: int = 64,
                  return_logprobs: bool = False):
        """Generate for already tokenised prompts on the calling thread; prompts that do not fit yield empty results."""
        stop_ids = set(self._task_mgr.tokenizer.stop_ids)
        tasks: List[Optional[Task]] = []
        for ids in prompt_ids_list:
            room = self.max_seq_len - len(ids)
            budget = room if max_tokens is None else min(max_tokens, room)
            if len(ids) >= self.max_seq_len or budget <= 0:
                tasks.append(None)
                continue
            self._batch_serial += 1  # ids must sort alike on every rank of a tensor-parallel replica: a counter, not a random id
            name = f"batch_{self._batch_serial:012d}" if self._control is not None else f"batch_{uuid.uuid4().hex[:8]}"
            task = Task(name, list(ids), budget, temperature, top_p, top_k, frequency_penalty, rep_window)
            if not self._task_cache.task_alloc(task.task_id, task.prompt_ids):
                tasks.append(None)
                continue
            task.input_tokens = len(task.prompt_ids)
            self._metrics.register(task.task_id)
            tasks.append(task)
        try:
            live = [t for t in tasks if t is not None]
            while live:
                before = sum(t.prefill_pos or 0 for t in live)
                decoded, _ = self._step(live, return_logprobs=return_logprobs)
                produced = {id(t) for t in decoded}
                # a request without a token this step stays only while its (chunked) prefill is still advancing
                waiting = [t for t in live if id(t) not in produced and self.chunked_prefill and not t.prefill_done
                           and t.status != TaskStatus.ABORTED]
                if not decoded and sum(t.prefill_pos or 0 for t in waiting) == before:
                    waiting = []
                live = [t for t in live if (id(t) in produced and not t.is_finished(stop_ids)) or t in waiting]
        finally:
            for t in tasks:
                if t is not None:
                    self._metrics.mark_finished(t.task_id, t.input_tokens, t.output_tokens)
                    self._task_cache.task_free(t.task_id)
        if return_logprobs:
            return [([], []) if t is None else (list(t.output_ids), list(t.output_logprobs)) for t in tasks]
        return [[] if t is None else list(t.output_ids) for t in tasks]
