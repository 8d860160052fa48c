"""Process-group bring-up and the per-GPU process launcher.

One process per GPU over ``torch.distributed`` (NCCL on NVLink 5 / NVSwitch; Gloo for CPU tests).  Behaviour
mirrors ``astrai/parallel/setup.py:20-281``: an external launcher (torchrun, SLURM, hand-set RANK/WORLD_SIZE) is
detected and used as is; otherwise ranks are spawned locally, signals are forwarded to the children and a child
failure terminates its siblings.  ``LOCAL_DEVICE``, ``LOCAL_RANK``, ``WORLD_SIZE``, ``MASTER_ADDR/PORT`` are exported
for each rank.
"""

from __future__ import annotations

import datetime
import functools
import logging
import os
import signal
import socket
import threading
from contextlib import contextmanager
from typing import Callable, Optional

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from astrai_b200.signal_handler import install_early_signal_handlers

logger = logging.getLogger(__name__)


def find_free_port() -> str:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return str(s.getsockname()[1])


def get_world_size() -> int:
    return dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1


def get_rank() -> int:
    return dist.get_rank() if dist.is_available() and dist.is_initialized() else 0


def get_current_device() -> str:
    dev = os.environ.get("LOCAL_DEVICE")
    if dev is None:
        dev = "cuda:0" if torch.cuda.is_available() else "cpu"
    return dev


def _device_for(device_type: str, local_rank: int) -> torch.device:
    return torch.device("cpu") if device_type == "cpu" else torch.device(device_type, local_rank)


@contextmanager
def setup_parallel(rank: int, world_size: int, local_rank: int, backend: str = "nccl",
                   master_addr: str = "127.0.0.1", master_port: str = "29500", device_type: str = "cuda",
                   timeout_s: Optional[float] = None):
    """Initialise (and on exit destroy) the WORLD process group for this rank."""
    if dist.is_available() and dist.is_initialized():
        yield dist.group.WORLD
        return
    device = _device_for(device_type, local_rank)
    os.environ["LOCAL_RANK"] = str(local_rank)
    os.environ["WORLD_SIZE"] = str(world_size)
    os.environ["LOCAL_DEVICE"] = str(device)
    if device.type == "cuda" and torch.cuda.is_available():
        torch.cuda.set_device(device)
    if world_size <= 1:
        yield None
        return
    os.environ["MASTER_ADDR"] = master_addr
    os.environ["MASTER_PORT"] = str(master_port)
    os.environ.setdefault("RANK", str(rank))
    kwargs = dict(rank=rank, world_size=world_size, backend=backend)
    if backend == "nccl":
        kwargs["device_id"] = device
    if timeout_s is not None:
        kwargs["timeout"] = datetime.timedelta(seconds=timeout_s)
    dist.init_process_group(**kwargs)
    try:
        yield dist.group.WORLD
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def only_on_rank(rank: int, sync: bool = False):
    """Decorator: run the function on one rank only (others get ``None``), optionally followed by a barrier."""

    def deco(fn):
        @functools.wraps(fn)
        def wrapper(*a, **k):
            out = fn(*a, **k) if get_rank() == rank else None
            if sync and dist.is_available() and dist.is_initialized():
                dist.barrier()
            return out

        return wrapper

    return deco


def _rank_main(rank: int, world_size: int, backend: str, addr: str, port: str, device_type: str, func: Callable, kwargs: dict):
    install_early_signal_handlers()
    with setup_parallel(rank, world_size, rank, backend, addr, port, device_type):
        func(**kwargs)


def launched_externally() -> bool:
    if dist.is_available() and dist.is_torchelastic_launched():
        return True
    env = os.environ
    return "LOCAL_WORLD_SIZE" in env or ("RANK" in env and "WORLD_SIZE" in env)


def _run_under_external_launcher(func, backend, addr, port, device_type, kwargs):
    install_early_signal_handlers()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    with setup_parallel(rank, world, local, backend, os.environ.get("MASTER_ADDR", addr),
                        os.environ.get("MASTER_PORT", port), device_type):
        func(**kwargs)


def _spawn_local(func, world_size, backend, addr, port, device_type, start_method, kwargs):
    args = (world_size, backend, addr, port, device_type, func, kwargs)
    if world_size == 1:
        _rank_main(0, *args)
        return
    install_early_signal_handlers()
    ctx = mp.start_processes(_rank_main, args=args, nprocs=world_size, start_method=start_method, join=False)
    stop = threading.Event()

    def terminate_children():
        for p in ctx.processes:
            if p.is_alive():
                p.terminate()

    def on_signal(signum, _frame):
        logger.warning("launcher pid %d got %s: forwarding to ranks", os.getpid(), signal.Signals(signum).name)
        stop.set()
        terminate_children()

    previous = {s: signal.signal(s, on_signal) for s in (signal.SIGTERM, signal.SIGINT)}
    try:
        while not stop.is_set() and not ctx.join(timeout=1.0):
            pass
    except BaseException:
        terminate_children()
        raise
    finally:
        for s, h in previous.items():
            if callable(h) and h is not on_signal:
                signal.signal(s, h)
        for p in ctx.processes:  # a rank that ignores SIGTERM (or is wedged) is killed after a grace period
            p.join(timeout=15 if stop.is_set() else None)
            if p.is_alive():
                p.kill()
                p.join()


class LaunchStrategy:
    """How ``func`` gets its ranks (the reference's ``LaunchStrategy`` classes, ``astrai/parallel/setup.py:138-247``)."""

    def __init__(self, world_size: int, backend: str, master_addr: str, master_port: str, device_type: str, start_method: str = "spawn"):
        self.world_size, self.backend, self.master_addr, self.master_port = world_size, backend, master_addr, str(master_port)
        self.device_type, self.start_method = device_type, start_method

    def launch(self, func: Callable, **kwargs):
        raise NotImplementedError


class TorchrunStrategy(LaunchStrategy):
    """The ranks exist already (torchrun, SLURM, Kubernetes set RANK / WORLD_SIZE / LOCAL_RANK): join them."""

    def launch(self, func: Callable, **kwargs):
        _run_under_external_launcher(func, self.backend, self.master_addr, self.master_port, self.device_type, kwargs)


class LocalStrategy(LaunchStrategy):
    """Start ``world_size`` processes on this node (none for a world of one), forward stop signals to them, reap them."""

    def launch(self, func: Callable, **kwargs):
        _spawn_local(func, self.world_size, self.backend, self.master_addr, self.master_port, self.device_type, self.start_method, kwargs)


def launch_strategy(world_size: int, backend: str = "nccl", master_addr: str = "127.0.0.1", master_port: Optional[str] = None,
                    device_type: str = "cuda", start_method: str = "spawn") -> LaunchStrategy:
    port = str(master_port) if master_port is not None else find_free_port()
    kind = TorchrunStrategy if launched_externally() else LocalStrategy
    return kind(world_size, backend, master_addr, port, device_type, start_method)


def spawn_parallel_fn(func: Callable, world_size: int, backend: str = "nccl", master_addr: str = "127.0.0.1",
                      master_port: Optional[str] = None, device_type: str = "cuda", start_method: str = "spawn", **kwargs):
    """Run ``func(**kwargs)`` on ``world_size`` ranks (here, or inside an already-launched rank)."""
    launch_strategy(world_size, backend, master_addr, master_port, device_type, start_method).launch(func, **kwargs)
