"""Rank-failure detection on the host: per-rank heartbeats in the process group's key-value store and a watchdog thread.

Liveness and progress are separate.  A daemon thread on every rank publishes ``(progress step, wall time)`` under
``hb/<rank>`` every ``interval_s`` - so a long step, a validation pass or a checkpoint write never makes a healthy
rank look dead - and reads its peers' entries: a peer is dead when its entry is older than ``timeout_s`` or when it
has announced its own exit with :meth:`Heartbeat.leave`.  :meth:`Heartbeat.beat` only advances the progress step.
The training loop asks :meth:`Heartbeat.check` before every micro-batch, and before a micro-batch that will issue
collectives it calls :meth:`Heartbeat.rendezvous`: every rank adds itself to a store counter and waits until all
ranks have arrived or one is known dead, so no survivor walks into a collective that a dead rank will never join.
A dead peer raises :class:`RankFailure` on the survivors *between* launches; what follows (emergency checkpoint, exit)
must then not communicate: see ``CheckpointCallback`` and ``Trainer``.  Nothing here touches a GPU; failures are
injected on the host in the tests (a rank that stops beating, leaves, or raises).

The reference has no heartbeat or watchdog: it relies on signal forwarding and on the process-group timeout
(``astrai/parallel/setup.py:209-247``).
"""

from __future__ import annotations

import logging
import threading
import time
from typing import Callable, Dict, List, Optional

import torch.distributed as dist

logger = logging.getLogger(__name__)


class RankFailure(RuntimeError):
    def __init__(self, ranks: List[int], why: str):
        super().__init__(f"rank(s) {ranks} {why}")
        self.ranks = ranks


class Heartbeat:
    """``store`` is any c10d store (TCPStore / FileStore / HashStore); by default the default group's store."""

    def __init__(self, rank: int, world_size: int, store=None, timeout_s: float = 60.0, interval_s: float = 1.0,
                 on_failure: Optional[Callable[[List[int]], None]] = None, prefix: str = "hb"):
        if store is None:
            store = dist.distributed_c10d._get_default_store()
        self.rank, self.world_size, self.store = rank, world_size, store
        self.timeout_s, self.interval_s, self.on_failure, self.prefix = float(timeout_s), float(interval_s), on_failure, prefix
        self._dead: Dict[int, str] = {}
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self._lock = threading.Lock()
        self._left = False
        self.step = 0

    # -- this rank -------------------------------------------------------------------------------------------------------
    def beat(self, step: Optional[int] = None):
        """Advance the progress step (call once per optimizer step) and publish it at once."""
        self.step = self.step + 1 if step is None else int(step)
        self._publish()

    def _publish(self):
        if not self._left:
            self.store.set(f"{self.prefix}/{self.rank}", f"{self.step} {time.time():.3f}")

    def leave(self, reason: str = "left"):
        """Announce an orderly exit so that the peers stop waiting at once instead of after ``timeout_s``."""
        self._left = True
        self.store.set(f"{self.prefix}/{self.rank}", f"-1 {time.time():.3f} {reason}")

    # -- the peers ---------------------------------------------------------------------------------------------------------
    def _read(self, peer: int):
        try:
            if hasattr(self.store, "check") and not self.store.check([f"{self.prefix}/{peer}"]):
                return None
            raw = self.store.get(f"{self.prefix}/{peer}").decode()
        except Exception:  # noqa: BLE001 - a store that went away is itself a failure signal, handled by the caller
            return None
        parts = raw.split(" ", 2)
        return int(parts[0]), float(parts[1]), (parts[2] if len(parts) > 2 else "")

    def scan(self) -> Dict[int, str]:
        """One pass over the peers; returns {rank: reason} of the ones considered dead so far."""
        now = time.time()
        for peer in range(self.world_size):
            if peer == self.rank or peer in self._dead:
                continue
            got = self._read(peer)
            if got is None:
                continue  # has not started beating yet: start-up is covered by the rendezvous timeout
            step, stamp, reason = got
            if step < 0:
                why = f"announced its exit ({reason})"
            elif now - stamp > self.timeout_s:
                why = f"has not beaten for {now - stamp:.1f} s (last step {step})"
            else:
                continue
            with self._lock:
                if peer in self._dead:
                    continue  # the other scanner (the thread, or a caller of scan) reported it a moment ago
                self._dead[peer] = why
            logger.error("heartbeat: rank %d %s", peer, why)
            if self.on_failure is not None:
                self.on_failure([peer])
        with self._lock:
            return dict(self._dead)

    def _loop(self):
        while not self._stop.wait(self.interval_s):
            try:
                self._publish()  # liveness: this process is up, whatever its main thread is busy with
                self.scan()
            except Exception as exc:  # noqa: BLE001
                logger.warning("heartbeat scan failed: %s", exc)

    def start(self) -> "Heartbeat":
        self.beat(0)
        self._thread = threading.Thread(target=self._loop, name="astrai-heartbeat", daemon=True)
        self._thread.start()
        return self

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2 * self.interval_s + 1)

    def dead_ranks(self) -> List[int]:
        with self._lock:
            return sorted(self._dead)

    def check(self):
        """Raise :class:`RankFailure` if a peer is known to be dead.  Call between steps, before the next launch."""
        with self._lock:
            dead = dict(self._dead)
        if dead:
            ranks = sorted(dead)
            raise RankFailure(ranks, "; ".join(dead[r] for r in ranks))

    def rendezvous(self, tag: str, poll_s: float = 0.002):
        """Host-side agreement before a launch that communicates: returns once every rank has reached ``tag``, raises
        :class:`RankFailure` as soon as a peer is known dead instead.  One store add plus a few reads per call."""
        key = f"{self.prefix}/rv/{tag}"
        arrived = self.store.add(key, 1)
        waited = 0.0
        while arrived < self.world_size:
            self.check()
            time.sleep(poll_s)
            waited += poll_s
            if waited >= self.interval_s:  # do not rely on the thread alone while blocked here
                waited = 0.0
                self.scan()
            arrived = self.store.add(key, 0)
        self.check()


class HeartbeatCallback:
    """Trainer callback: progress beat after every optimizer step, failure check before every micro-batch, host-side
    rendezvous before a micro-batch that communicates, orderly leave on exit / error.

    On a failure the context gets ``failed_ranks`` (the checkpoint callback and the trainer then avoid every collective),
    a stop is requested and :class:`RankFailure` is raised from ``on_batch_begin``.
    """

    def __init__(self, timeout_s: float = 60.0, interval_s: float = 1.0, every_micro_batch: bool = False):
        self.timeout_s, self.interval_s, self.every_micro_batch = timeout_s, interval_s, every_micro_batch
        self.hb: Optional[Heartbeat] = None
        self._micro = 0

    def _failed(self, context, ranks):
        context.failed_ranks = sorted(set(getattr(context, "failed_ranks", None) or []) | set(ranks))
        context.request_stop()

    def on_train_begin(self, context):
        if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
            self.hb = Heartbeat(dist.get_rank(), dist.get_world_size(), timeout_s=self.timeout_s, interval_s=self.interval_s,
                                on_failure=lambda ranks: self._failed(context, ranks)).start()

    def on_batch_begin(self, context):
        if self.hb is None:
            return
        self._micro += 1
        try:
            self.hb.check()
            ex = context.executor
            # data-parallel modes communicate on the micro-batch that closes an accumulation window only; model-parallel
            # modes (tp / cp / ep / pp) in every forward pass
            if self.every_micro_batch or ex.sync_gradients or getattr(ex, "communicates_every_micro_batch", False):
                self.hb.rendezvous(str(self._micro))
        except RankFailure as exc:
            self._failed(context, exc.ranks)
            raise

    def on_optimizer_step(self, context):
        if self.hb is not None:
            self.hb.beat()

    def on_error(self, context):
        if self.hb is not None:
            self.hb.leave("error")

    def on_train_end(self, context):
        if self.hb is not None:
            self.hb.leave("finished")
            self.hb.stop()

    def on_epoch_begin(self, context): ...
    def on_epoch_end(self, context): ...
    def on_batch_end(self, context): ...
