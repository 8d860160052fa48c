"""Rank-failure detection on the host: per-rank heartbeats in the process group's key-value store and a watchdog thread.

Every rank publishes ``(step, wall time)`` under ``hb/<rank>`` after each optimizer step; a daemon thread on every rank
reads its peers' entries every ``interval_s`` and declares a peer dead when its heartbeat is older than ``timeout_s``
(or when it has announced its own exit with :meth:`Heartbeat.leave`).  The training loop asks :meth:`Heartbeat.check`
before launching the next step: a dead peer raises :class:`RankFailure` on the survivors *between* steps - with no
kernel or collective of theirs in flight - so they can write an emergency checkpoint and exit instead of sitting in a
collective until its timeout.  Nothing here touches a GPU; failures are injected on the host in the tests (a rank that
stops beating, leaves, or raises).

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
        self.step = 0

    # -- this rank -------------------------------------------------------------------------------------------------------
    def beat(self, step: Optional[int] = None):
        """Publish "alive at `step`" (call once per optimizer step)."""
        self.step = self.step + 1 if step is None else int(step)
        self.store.set(f"{self.prefix}/{self.rank}", f"{self.step} {time.time():.3f}")

    def leave(self, reason: str = "left"):
        """Announce an orderly exit so that the peers stop waiting at once instead of after ``timeout_s``."""
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
                self._dead[peer] = why
            logger.error("heartbeat: rank %d %s", peer, why)
            if self.on_failure is not None:
                self.on_failure([peer])
        with self._lock:
            return dict(self._dead)

    def _loop(self):
        while not self._stop.wait(self.interval_s):
            try:
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

    def check(self):
        """Raise :class:`RankFailure` if a peer is known to be dead.  Call between steps, before the next launch."""
        with self._lock:
            dead = dict(self._dead)
        if dead:
            ranks = sorted(dead)
            raise RankFailure(ranks, "; ".join(dead[r] for r in ranks))


class HeartbeatCallback:
    """Trainer callback: beat after every optimizer step, check before every micro-batch, leave on exit / error.
    A detected failure requests a stop (emergency checkpoint through the trainer's usual path) and re-raises."""

    def __init__(self, timeout_s: float = 60.0, interval_s: float = 1.0):
        self.timeout_s, self.interval_s = timeout_s, interval_s
        self.hb: Optional[Heartbeat] = None

    def on_train_begin(self, context):
        if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
            self.hb = Heartbeat(dist.get_rank(), dist.get_world_size(), timeout_s=self.timeout_s, interval_s=self.interval_s,
                                on_failure=lambda ranks: context.request_stop()).start()

    def on_batch_begin(self, context):
        if self.hb is not None:
            self.hb.check()

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
