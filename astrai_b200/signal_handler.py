"""SIGTERM / SIGINT -> graceful stop of the training loop.

Reference behaviour (``astrai/signal_handler.py:8-53``): handlers are installed
as early as possible in every rank; a signal that arrives before the training
context exists is remembered and replayed when the context registers.
"""

import logging
import os
import signal
import threading

logger = logging.getLogger(__name__)

_SIGNALS = (signal.SIGTERM, signal.SIGINT)
_pending = threading.Event()
_context = None


def _on_signal(signum, _frame):
    logger.warning("pid %d got %s: asking the trainer to stop", os.getpid(), signal.Signals(signum).name)
    _pending.set()
    ctx = _context
    if ctx is not None:
        ctx.request_stop()


def _unblock():
    try:
        blocked = set(_SIGNALS) & signal.pthread_sigmask(signal.SIG_BLOCK, set())
        if blocked:
            signal.pthread_sigmask(signal.SIG_UNBLOCK, blocked)
    except (AttributeError, OSError):
        pass


def install_early_signal_handlers():
    for s in _SIGNALS:
        signal.signal(s, _on_signal)
    _unblock()


def register_signal_handlers(context):
    global _context
    _context = context
    for s in _SIGNALS:
        signal.signal(s, _on_signal)
    if _pending.is_set():
        logger.warning("a stop signal arrived during start-up; stopping")
        context.request_stop()


def unregister_signal_handlers():
    global _context
    _context = None
    _pending.clear()
