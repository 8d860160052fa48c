"""The training loop.

Control flow of the reference (``astrai/trainer/trainer.py:61-134``): per micro-batch ``accumulate -> strategy ->
loss / accum -> backward -> on_batch_end``; on the micro-batch that closes an accumulation window
``on_optimizer_step -> optimizer.step -> strategy.on_optimizer_step -> zero_grad -> scheduler.step``.  A stop signal
or an exception triggers ``on_error`` (emergency checkpoint) and ``on_train_end`` always runs.

Differences: the loss is not read back to the host per micro-batch (it is kept as a tensor and converted on first
read), and on the flat runtime the ``1/accum`` factor is handed to the fused projection + loss kernel instead of being
multiplied into the graph.
"""

from __future__ import annotations

import logging
import time
from typing import List, Optional

import torch
import torch.distributed as dist

from astrai_b200.utils import trace
from astrai_b200 import ops
from astrai_b200.config import TrainConfig
from astrai_b200.parallel.setup import spawn_parallel_fn
from astrai_b200.signal_handler import register_signal_handlers, unregister_signal_handlers
from astrai_b200.trainer.train_callback import CallbackFactory, TrainCallback
from astrai_b200.trainer.train_context import TrainContext, TrainContextBuilder

logger = logging.getLogger(__name__)


class Trainer:
    def __init__(self, train_config: TrainConfig, callbacks: Optional[List[TrainCallback]] = None):
        self.train_config = train_config
        self.callbacks = self._default_callbacks() + list(callbacks or [])

    def _default_callbacks(self) -> List[TrainCallback]:
        c = self.train_config
        # Clipping runs first so that the metric log and the progress bar of a step show that step's gradient norm
        # (the reference lists it last, which makes the logged norm lag one step behind).
        watch = []
        if c.heartbeat_timeout_s and c.nprocs > 1:
            # first in the list: its failure check runs before any other callback of a micro-batch
            watch = [CallbackFactory.create("heartbeat", timeout_s=c.heartbeat_timeout_s, interval_s=c.heartbeat_interval_s)]
        return watch + [
            CallbackFactory.create("gradient_checkpointing", modules=c.gradient_checkpointing_modules),
            CallbackFactory.create("gradient_clipping", c.max_grad_norm),
            CallbackFactory.create("checkpoint", c.ckpt_dir, c.ckpt_interval),
            CallbackFactory.create("metric", ckpt_dir=c.ckpt_dir, save_interval=c.ckpt_interval, metrics=c.metrics,
                                   val_step=c.val_step),
            CallbackFactory.create("progress_bar", c.n_epoch),
        ]

    def _fire(self, hook: str, context: TrainContext):
        for cb in self.callbacks:
            fn = getattr(cb, hook, None)
            if fn:
                fn(context)

    def _micro_batch(self, context: TrainContext, batch):
        ex = context.executor
        scale = 1.0 / ex.grad_accum_steps
        flat = getattr(ex, "engine", None) is not None
        self._fire("on_batch_begin", context)
        if hasattr(ex, "pipeline_step"):
            # pipeline parallelism: forward and backward of the batch's pieces interleave across the stages inside the call
            with trace.range("pipeline"):
                out = ex.pipeline_step(context.model, batch, scale, strategy=context.strategy)
            loss = out["loss"]
        elif flat:
            # promise the loss gradient so the fused head bakes 1/accum into dX and accumulates dW in place
            with trace.range("forward"), ops.assume_loss_grad(scale):
                out = context.strategy(batch)
            loss = out["loss"]
            with trace.range("backward"):
                ex.backward(loss, torch.full_like(loss, scale))
        else:
            with trace.range("forward"):
                out = context.strategy(batch)
            loss = out["loss"]
            with trace.range("backward"):
                ex.backward(loss * scale)
        context.loss = loss.detach()
        context.metrics = out["metrics"]
        context.consumed_samples += context.config.batch_per_device * context.samples_world
        self._fire("on_batch_end", context)
        if ex.sync_gradients:
            self._fire("on_optimizer_step", context)
            with trace.range("optimizer"):
                context.optimizer.step()
            context.strategy.on_optimizer_step()
            context.optimizer.zero_grad()
            if context.scheduler:
                context.scheduler.step()

    def _trainer_loop(self, param_path: Optional[str] = None, resume: bool = False):
        context = TrainContextBuilder(self.train_config).with_param_path(param_path, resume=resume).build()
        register_signal_handlers(context)
        ex = context.executor
        self._fire("on_train_begin", context)
        try:
            context.model.train()
            for epoch in range(context.epoch, context.config.n_epoch):
                if context.stop_requested:
                    break
                context.epoch = epoch
                self._fire("on_epoch_begin", context)
                for batch in context.dataloader:
                    if context.stop_requested:
                        break
                    with ex.accumulate(context.model):
                        self._micro_batch(context, batch)
                self._fire("on_epoch_end", context)
            if context.stop_requested:
                logger.warning("Training interrupted by signal, saving emergency checkpoint...")
                self._fire("on_error", context)
        except Exception as exc:
            logger.error("Training failed: %s", exc, exc_info=True)
            self._fire("on_error", context)
            raise
        finally:
            self._fire("on_train_end", context)
            # a barrier would wait for a rank that is known to be gone
            if ex.use_distributed and dist.is_initialized() and not getattr(context, "failed_ranks", None):
                dist.barrier()
            unregister_signal_handlers()
        return context

    def train(self, param_path: Optional[str] = None, resume: bool = False):
        c = self.train_config
        spawn_parallel_fn(self._trainer_loop, backend=c.backend, world_size=c.nprocs, master_addr=c.master_addr,
                          master_port=c.master_port, device_type=c.device_type, start_method=c.start_method,
                          param_path=param_path, resume=resume)
