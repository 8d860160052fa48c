"""Trainer callbacks: gradient clipping, activation checkpointing, checkpoints, progress bar, metric log.

Hook names, default callbacks, file names and cadence follow ``astrai/trainer/train_callback.py:33-375``:
checkpoints in ``<ckpt_dir>/epoch_{E}_step_{S}``, metric events (one JSON object per line) in ``metric.jsonl`` of the
same directory, validation every ``val_step`` optimizer steps, values averaged over ranks.
"""

from __future__ import annotations

import json
import logging
import os
import sys
import time
from functools import partial
from pathlib import Path
from typing import IO, Callable, List, Optional, Protocol, runtime_checkable

import torch
import torch.distributed as dist
import torch.nn as nn
from torch.utils.checkpoint import checkpoint as activation_checkpoint

from astrai_b200.factory import BaseFactory
from astrai_b200.parallel.setup import get_current_device, get_rank
from astrai_b200.serialization import Checkpoint
from astrai_b200.trainer import metric_util as mu

logger = logging.getLogger(__name__)


@runtime_checkable
class TrainCallback(Protocol):
    def on_train_begin(self, context): ...
    def on_train_end(self, context): ...
    def on_epoch_begin(self, context): ...
    def on_epoch_end(self, context): ...
    def on_batch_begin(self, context): ...
    def on_batch_end(self, context): ...
    def on_optimizer_step(self, context): ...
    def on_error(self, context): ...


class CallbackFactory(BaseFactory[TrainCallback]):
    pass


@CallbackFactory.register("gradient_clipping")
class GradientClippingCallback(TrainCallback):
    """Clips to ``max_grad_norm`` (None = only the flat runtime's averaging scale is applied, nothing is measured)."""

    def __init__(self, max_grad_norm: Optional[float]):
        self.max_grad_norm = max_grad_norm

    def on_optimizer_step(self, context):
        if self.max_grad_norm is None:
            return
        context.grad_norm = context.executor.clip_grad_norm(context.model, self.max_grad_norm)


@CallbackFactory.register("gradient_checkpointing")
class GradientCheckpointingCallback(TrainCallback):
    """Recompute the activations of the listed module types in backward instead of keeping them."""

    def __init__(self, modules: Optional[List[type]] = None):
        self.modules = tuple(modules or ())

    def _wrap(self, module: nn.Module):
        if self.modules and isinstance(module, self.modules) and not hasattr(module, "_plain_forward"):
            plain = module.forward
            module._plain_forward = plain
            module.forward = lambda *a, **k: activation_checkpoint(plain, *a, use_reentrant=False, **k)

    @staticmethod
    def _unwrap(module: nn.Module):
        if hasattr(module, "_plain_forward"):
            module.forward = module._plain_forward
            del module._plain_forward

    def on_train_begin(self, context):
        if self.modules:
            context.model.apply(self._wrap)

    def on_train_end(self, context):
        context.model.apply(self._unwrap)


@CallbackFactory.register("checkpoint")
class CheckpointCallback(TrainCallback):
    extra_keys = ("optimizer", "scheduler")

    def __init__(self, save_dir: str, interval: int, weight_only: bool = False,
                 save_extra_fn: Optional[Callable] = None):
        self.save_dir, self.interval, self.weight_only = save_dir, interval, weight_only
        self.save_extra_fn = save_extra_fn or CheckpointCallback.save_extra
        self.last_ckpt_step = None

    @staticmethod
    def save_extra(context) -> dict:
        out = {}
        for name in CheckpointCallback.extra_keys:
            obj = getattr(context, name, None)
            if obj:
                out[name] = obj.state_dict()
        return out

    def _save_without_peers(self, context, dead: List[int]):
        """Emergency save while ``dead`` ranks are gone: nothing here may communicate (no barrier, no gather).

        ONE survivor writes the usual directory from its local copy of the weights: the first to create
        ``<dir>.writer`` (an exclusive create on the shared file system - survivors may disagree about who is still
        alive, because a rank that has finished its own emergency save and left looks gone as well).  Every executor whose
        parameters are replicated or locally complete can give one; a torch-FSDP2 model cannot, its save is skipped)
        with ``emergency`` / ``failed_ranks`` in ``meta.json``.  A sharded optimizer is not gathered: every survivor
        writes its own shard to ``<dir>.shards/optimizer.rank<r>.pt`` (the dead ranks' shards are lost, so the directory
        holds no ``optimizer.pt`` and does not count as complete for an automatic resume; the weights are intact).
        """
        self.last_ckpt_step = context.optimizer_step
        rank, world = get_rank(), context.world_size
        survivors = [r for r in range(world) if r not in set(dead)]
        path = os.path.join(self.save_dir, f"epoch_{context.epoch}_step_{context.optimizer_step}")
        extra = {}
        if not self.weight_only:
            sched = getattr(context, "scheduler", None)
            if sched:
                extra["scheduler"] = sched.state_dict()
            opt = getattr(context, "optimizer", None)
            if opt:
                try:
                    osd = opt.state_dict(gather=False)
                except TypeError:
                    osd = opt.state_dict()
                if isinstance(osd, dict) and osd.get("flat_layout") == "shard":
                    shard_dir = Path(path + ".shards")
                    shard_dir.mkdir(parents=True, exist_ok=True)
                    torch.save(osd, shard_dir / f"optimizer.rank{rank}.pt")
                else:
                    extra["optimizer"] = osd
        if not survivors or (Path(path) / "meta.json").exists():
            return
        state_dict = context.executor.local_state_dict(context.model)
        if state_dict is None:
            logger.error("emergency checkpoint: this executor cannot produce the weights without its peers; nothing written")
            return
        os.makedirs(self.save_dir, exist_ok=True)
        try:
            os.close(os.open(path + ".writer", os.O_CREAT | os.O_EXCL | os.O_WRONLY))
        except FileExistsError:
            return  # another survivor is writing (or has written) this step
        try:
            meta = dict(context.config.to_dict(), emergency=True, failed_ranks=sorted(dead), written_by_rank=rank)
            context.checkpoint = Checkpoint(state_dict=state_dict, epoch=context.epoch, consumed_samples=context.consumed_samples,
                                            config=context.model_config, extra=extra, meta=meta)
            context.checkpoint.save(path)
        finally:
            os.unlink(path + ".writer")

    def _save(self, context):
        dead = getattr(context, "failed_ranks", None)
        if dead:
            return self._save_without_peers(context, dead)
        self.last_ckpt_step = context.optimizer_step
        extra = {} if self.weight_only else self.save_extra_fn(context)  # collective for sharded optimizers
        with context.executor.checkpoint_context(context.model) as state_dict:
            if state_dict is None:
                return
            path = os.path.join(self.save_dir, f"epoch_{context.epoch}_step_{context.optimizer_step}")
            context.checkpoint = Checkpoint(state_dict=state_dict, epoch=context.epoch,
                                            consumed_samples=context.consumed_samples, config=context.model_config,
                                            extra=extra, meta=context.config.to_dict())
            context.checkpoint.save(path)

    def on_train_begin(self, context):
        self.last_ckpt_step = context.optimizer_step

    def on_batch_end(self, context):
        if context.optimizer_step - self.last_ckpt_step >= self.interval:
            self._save(context)

    def on_train_end(self, context):
        if context.optimizer_step != self.last_ckpt_step:
            self._save(context)

    def on_error(self, context):
        self._save(context)


@CallbackFactory.register("heartbeat")
class _HeartbeatCallback(TrainCallback):
    """Rank-failure detection through store heartbeats (see :mod:`astrai_b200.parallel.watchdog`)."""

    def __new__(cls, *args, **kwargs):
        from astrai_b200.parallel.watchdog import HeartbeatCallback

        return HeartbeatCallback(*args, **kwargs)


@CallbackFactory.register("progress_bar")
class ProgressBarCallback(TrainCallback):
    def __init__(self, num_epoch: int, log_interval: int = 100, file: Optional[IO[str]] = None):
        self.num_epoch, self.log_interval, self.file = num_epoch, log_interval, file
        self.progress_bar = None

    def on_epoch_begin(self, context):
        if get_rank() != 0:
            return
        from tqdm import tqdm

        self.progress_bar = tqdm(total=len(context.dataloader) // context.executor.grad_accum_steps,
                                 desc=f"Epoch {context.epoch + 1}/{self.num_epoch}", dynamic_ncols=True,
                                 file=self.file or sys.stdout)

    def on_optimizer_step(self, context):
        if get_rank() != 0 or self.progress_bar is None:
            return
        post = {"step": f"{context.optimizer_step:d}", "loss": f"{context.loss:.4f}",
                "lr": f"{context.optimizer.param_groups[-1]['lr']:.2e}"}
        if context.grad_norm is not None:
            post["grad_norm"] = f"{context.grad_norm:.2f}"
        if context.val_loss is not None:
            post["val_loss"] = f"{context.val_loss:.4f}"
        self.progress_bar.set_postfix(post)
        self.progress_bar.update(1)

    def on_epoch_end(self, context):
        if self.progress_bar is not None:
            self.progress_bar.close()


@CallbackFactory.register("metric")
class MetricCallback(TrainCallback):
    def __init__(self, ckpt_dir: str, save_interval: int, metrics: Optional[List[str]] = None, val_step: int = 0):
        self.ckpt_dir = Path(ckpt_dir) if ckpt_dir else Path.cwd() / "checkpoint"
        self.save_interval, self.val_step = save_interval, val_step
        self.metrics = metrics or ["loss", "lr"]
        self.log_cache: List[dict] = []
        self.last_log_flush_step = None
        self._next_val_step = 0
        moe = lambda key: partial(mu.ctx_get_moe_metric, key=key)  # noqa: E731
        self._getters = {
            "loss": mu.ctx_get_loss, "lr": mu.ctx_get_lr, "val_loss": mu.ctx_get_val_loss,
            "grad_norm": mu.ctx_get_grad_norm, "grad_snr": mu.ctx_get_grad_snr, "moe_aux_loss": moe("aux_loss"),
            "router_entropy": moe("router_entropy"), "dead_expert_fraction": moe("dead_expert_fraction"),
            "load_imbalance_mean": moe("load_imbalance_mean"), "load_imbalance_max": moe("load_imbalance_max"),
        }

    def _collect(self, context, names) -> dict:
        values = dict(context.metrics.items()) if context.metrics else {}
        for n in names:
            fn = self._getters.get(n)
            v = fn(context) if fn is not None else None
            if v is not None:
                values[n] = v
        keep = (set(context.metrics or ()) | set(names)) - {"*"}
        out = {k: values[k] for k in keep if k in values}
        if context.world_size > 1 and dist.is_initialized() and out:
            keys = sorted(out)
            t = torch.tensor([out[k] for k in keys], dtype=torch.float32, device=get_current_device())
            dist.all_reduce(t)
            out.update(zip(keys, (t / context.world_size).tolist()))
        return out

    def _append(self, kind: str, context, **extra):
        if get_rank() != 0:
            return
        self.log_cache.append({"type": kind, "timestamp": time.strftime("%Y-%m-%dT%H:%M:%S"), "epoch": context.epoch,
                               "step": context.optimizer_step, "consumed_samples": context.consumed_samples, **extra})

    def _validate(self, context) -> float:
        context.model.eval()
        total, batches = 0.0, 0
        staged = getattr(getattr(context, "executor", None), "pipeline_eval", None)  # pipeline stages compute the loss between them
        with torch.no_grad():
            for batch in context.val_dataloader:
                out = staged(context.model, batch) if staged is not None else context.strategy(batch)
                total += float(out["loss"].item())
                batches += 1
        context.model.train()
        if context.world_size > 1 and dist.is_initialized():
            t = torch.tensor([total, float(batches)], device=get_current_device())
            dist.all_reduce(t)
            return (t[0] / t[1].clamp(min=1)).item()
        return total / max(batches, 1)

    def _flush(self, epoch, step):
        if get_rank() != 0:
            return
        path = self.ckpt_dir / f"epoch_{epoch}_step_{step}" / "metric.jsonl"
        path.parent.mkdir(parents=True, exist_ok=True)
        with open(path, "w") as fh:
            for row in self.log_cache:
                fh.write(json.dumps(row) + "\n")

    def on_train_begin(self, context):
        self.last_log_flush_step = context.optimizer_step

    def on_optimizer_step(self, context):
        if "grad_snr" in self.metrics:
            context.grad_snr_tracker.update(context.model)
        if context.val_dataloader is not None and self.val_step > 0 and context.optimizer_step >= self._next_val_step:
            context.val_loss = self._validate(context)
            self._next_val_step = context.optimizer_step + self.val_step
            self._append("validation", context, val_loss=context.val_loss)
        self._append("step", context, **self._collect(context, [m for m in self.metrics if m != "val_loss"]))
        if context.optimizer_step - self.last_log_flush_step >= self.save_interval:
            self._flush(context.epoch, context.optimizer_step)
            self.last_log_flush_step = context.optimizer_step

    def on_epoch_end(self, context):
        self._append("epoch", context)

    def on_train_end(self, context):
        if self.last_log_flush_step is None or context.optimizer_step != self.last_log_flush_step:
            self._flush(context.epoch, context.optimizer_step)
            self.last_log_flush_step = context.optimizer_step

    def on_error(self, context):
        self._flush(context.epoch, context.optimizer_step)
