"""Everything one training run needs, and the builder that assembles it.

Build order and resume arithmetic follow ``astrai/trainer/train_context.py:99-337``: load a checkpoint or model
directory (HuggingFace layouts are converted), create the executor, build / place / wrap the model, restore
optimizer and scheduler, split off validation data, create resumable samplers, create the strategy (with frozen
reference / behaviour models where the objective needs them) and wire online rollout.
``optimizer_step = consumed_samples // (batch_per_device * world_size * grad_accum_steps)``.
"""

from __future__ import annotations

import logging
import threading
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Dict, Optional

import torch
import torch.nn as nn
from torch.utils.data import DataLoader, random_split

from astrai_b200.config import ConfigFactory, TrainConfig
from astrai_b200.data import RDSampler
from astrai_b200.parallel.executor import BaseExecutor, ExecutorFactory, create_ref_model
from astrai_b200.parallel.setup import get_current_device, get_rank, get_world_size
from astrai_b200.serialization import Checkpoint, adapt_config, convert_hf_weights, load_json, looks_like_hf_state_dict
from astrai_b200.trainer.metric_util import GradSNRTracker
from astrai_b200.trainer.strategy import BaseStrategy, StrategyFactory

logger = logging.getLogger(__name__)


class TrainContext:
    """Mutable state shared by the trainer loop and its callbacks."""

    def __init__(self, **kw):
        self.model: nn.Module = None
        self.strategy: BaseStrategy = None
        self.dataloader: DataLoader = None
        self.optimizer = None
        self.scheduler = None
        self.checkpoint: Optional[Checkpoint] = None
        self.config: TrainConfig = None
        self.model_config: dict = {}
        self.executor: BaseExecutor = None
        self.epoch = 0
        self.consumed_samples = 0
        self.metrics: Dict[str, float] = {}
        self.grad_norm: Optional[float] = None
        self.grad_snr_tracker = GradSNRTracker()
        self.val_dataloader: Optional[DataLoader] = None
        self.val_loss: Optional[float] = None
        self.world_size = 1
        self.rank = 0
        self.data_world = None  # ranks that draw different samples (set by the builder; None: every rank)
        self.kwargs: Dict[str, Any] = {}
        self._loss: Any = 0.0
        self._stop_event = threading.Event()
        for k, v in kw.items():
            setattr(self, k, v)

    # The loss of the last micro-batch stays a device tensor until somebody reads it.
    @property
    def loss(self) -> float:
        if isinstance(self._loss, torch.Tensor):
            self._loss = float(self._loss.detach().float().item())
        return self._loss

    @loss.setter
    def loss(self, value):
        self._loss = value

    @property
    def stop_requested(self) -> bool:
        return self._stop_event.is_set()

    def request_stop(self) -> None:
        self._stop_event.set()

    @property
    def optimizer_step(self) -> int:
        c = self.config
        return self.consumed_samples // (c.batch_per_device * self.samples_world * c.grad_accum_steps)

    @property
    def samples_world(self) -> int:
        """How many ranks contribute distinct samples to one micro-batch of the job: the world size, except that the
        ranks of a tensor- or context-parallel block share one batch."""
        return self.data_world if self.data_world else self.world_size


@dataclass
class _Preloaded:
    model_config: dict = field(default_factory=dict)
    state_dict: Optional[dict] = None
    epoch: int = 0
    consumed_samples: int = 0
    checkpoint: Optional[Checkpoint] = None


class TrainContextBuilder:
    def __init__(self, config: TrainConfig):
        self.config = config
        self._param_path: Optional[str] = None
        self._resume = False

    def with_param_path(self, param_path: Optional[str], resume: bool = False):
        self._param_path, self._resume = param_path, resume
        return self

    def build(self) -> TrainContext:
        pre = self._preload()
        executor = self._executor()
        ctx = TrainContext(world_size=get_world_size(), rank=get_rank(), config=self.config,
                           model_config=pre.model_config, executor=executor, epoch=pre.epoch,
                           consumed_samples=pre.consumed_samples, checkpoint=pre.checkpoint,
                           data_world=self._data_world())
        self._model(ctx, executor, pre)
        self._restore_optimizer(ctx)
        train_ds, val_ds = self._datasets()
        self._dataloaders(ctx, train_ds, val_ds)
        strategy_kwargs = self._strategy(ctx, executor)
        self._rollout(ctx, strategy_kwargs)
        return ctx

    # ---------------------------------------------------------------------------------------------------------------
    def _data_world(self) -> int:
        from astrai_b200.parallel.mesh import data_parallel_size

        c = self.config
        return data_parallel_size(c.parallel_mode, get_world_size(), c.tp_size, c.cp_size, c.ep_size, c.pp_size)

    def _executor(self) -> BaseExecutor:
        c = self.config
        mode = c.parallel_mode
        kw = dict(c.executor_kwargs)
        size = {"tp": c.tp_size, "cp": c.cp_size, "ep": c.ep_size, "pp": c.pp_size}.get(mode)
        if size is not None:
            import astrai_b200.parallel.model_parallel  # noqa: F401 - registers the tp / cp / ep executors

            kw.setdefault("size", size)
        if mode == "pp":  # the last stage computes the loss itself: it takes the objective's options from the strategy's
            if c.strategy not in ("seq", "sft", "dpo", "grpo"):
                raise ValueError(f"parallel_mode 'pp' trains the strategies 'seq', 'sft', 'dpo' and 'grpo' on prepared data, not {c.strategy!r}")
            kw.setdefault("label_smoothing", float(c.strategy_kwargs.get("label_smoothing", 0.0) or 0.0))
            kw.setdefault("aux_loss_coef", float(c.strategy_kwargs.get("moe_aux_loss_coef", c.moe_aux_loss_coef)))
        return ExecutorFactory.create(mode, grad_accum_steps=c.grad_accum_steps, **kw)

    def _preload(self) -> _Preloaded:
        c = self.config
        pre = _Preloaded(epoch=c.start_epoch, consumed_samples=c.start_samples * self._data_world())
        if self._param_path:
            root = Path(self._param_path)
            if (root / "config.json").exists():
                pre.model_config = adapt_config(load_json(root / "config.json"))
            ck = Checkpoint.load_any(self._param_path)
            if ck is not None:
                if ck.config:
                    ck.config = adapt_config(ck.config)
                if ck.state_dict and looks_like_hf_state_dict(ck.state_dict):
                    ck.state_dict = convert_hf_weights(ck.state_dict, ConfigFactory.load(ck.config or pre.model_config))
                pre.state_dict = ck.state_dict
                pre.model_config = ck.config or pre.model_config
                if self._resume:
                    per_step = c.batch_per_device * self._data_world() * c.grad_accum_steps
                    pre.epoch = ck.epoch
                    pre.consumed_samples = ck.consumed_samples // per_step * per_step
                    pre.checkpoint = ck
        if not pre.model_config:
            probe = c.model_fn()
            if hasattr(probe, "config"):
                pre.model_config = probe.config.to_dict()
            del probe
        return pre

    def _model(self, ctx: TrainContext, executor: BaseExecutor, pre: _Preloaded):
        c = self.config
        device = get_current_device()

        def before_wrap(model):
            model = model.to(device=device)
            if c.neftune_alpha and hasattr(model, "embed_tokens"):
                model.embed_tokens.set_neftune_alpha(c.neftune_alpha)
            if c.lora is not None:
                from astrai_b200.models.lora import inject_lora

                inject_lora(model, r=c.lora.r, alpha=c.lora.alpha, target_modules=set(c.lora.target_modules))
            if pre.state_dict is not None:
                model.load_state_dict(pre.state_dict, strict=False)
            return model

        def after_wrap(model):
            if c.compile_mode is not None:
                # torch.compile is kept for interface parity; the native path does not need it
                model = torch.compile(model, mode=c.compile_mode)
            return model

        ctx.model, ctx.optimizer, ctx.scheduler = executor.prepare(
            c.model_fn, c.optimizer_fn, c.scheduler_fn, before_wrap=before_wrap, after_wrap=after_wrap)

    def _restore_optimizer(self, ctx: TrainContext):
        extra = ctx.checkpoint.extra if ctx.checkpoint else None
        for name in ("optimizer", "scheduler"):
            if extra and name in extra and getattr(ctx, name, None) is not None:
                getattr(ctx, name).load_state_dict(extra[name])

    def _datasets(self):
        c = self.config
        if c.val_dataset is not None or c.val_split is None:
            return c.dataset, c.val_dataset
        n_val = max(1, int(len(c.dataset) * c.val_split))
        g = torch.Generator().manual_seed(c.random_seed)
        return random_split(c.dataset, [len(c.dataset) - n_val, n_val], generator=g)

    def _loader(self, dataset, epoch: int, start_iter: int, shuffle: bool = True) -> DataLoader:
        c = self.config
        # ranks of one tensor- / context-parallel block must draw the same samples: deal by data-parallel position
        dw = self._data_world()
        part = (get_rank() // max(get_world_size() // dw, 1), dw) if dw != get_world_size() else None
        sampler = RDSampler(dataset, start_epoch=epoch, start_iter=start_iter, seed=c.random_seed, shuffle=shuffle,
                            partition=part)
        kw = dict(dataset=dataset, batch_size=c.batch_per_device, sampler=sampler, num_workers=c.num_workers,
                  pin_memory=c.pin_memory and torch.cuda.is_available(), collate_fn=c.collate_fn)
        if c.num_workers > 0:
            kw["persistent_workers"] = c.persistent_workers
            if c.prefetch_factor is not None:
                kw["prefetch_factor"] = c.prefetch_factor
        return DataLoader(**kw)

    def _dataloaders(self, ctx: TrainContext, train_ds, val_ds):
        offset = ctx.consumed_samples // ctx.samples_world
        if self._resume and offset > 0:
            per_replica = -(-len(train_ds) // ctx.samples_world)
            if per_replica > 0:
                ctx.epoch = offset // per_replica
        ctx.dataloader = self._loader(train_ds, ctx.epoch, offset)
        if val_ds is not None:
            ctx.val_dataloader = self._loader(val_ds, 0, 0, shuffle=False)

    def _strategy(self, ctx: TrainContext, executor: BaseExecutor) -> dict:
        c = self.config
        kw = dict(c.strategy_kwargs)
        kw.setdefault("moe_aux_loss_coef", c.moe_aux_loss_coef)
        device = get_current_device()
        if c.strategy in ("dpo", "grpo", "online_grpo", "online_dpo"):
            kw["ref_model"] = create_ref_model(c.model_fn, executor=executor, model=ctx.model, device=device)
        if c.strategy in ("grpo", "online_grpo"):
            kw["old_model"] = create_ref_model(c.model_fn, executor=executor, model=ctx.model, device=device)
        stage = getattr(getattr(executor, "_pipe", None), "stage", None)
        if stage is not None and not stage.last:
            # pipeline stages: only the last one scores with the frozen models (building them was a collective: the weights
            # were gathered from every stage); the others give the memory back
            for name in ("ref_model", "old_model"):
                if name in kw:
                    kw[name] = None
        ctx.strategy = StrategyFactory.create(c.strategy, model=ctx.model, device=device, executor=executor, **kw)
        return kw

    def _rollout(self, ctx: TrainContext, strategy_kwargs: dict):
        c = self.config
        if not c.strategy.startswith("online_"):
            return
        if not ctx.strategy.supports_online():
            raise ValueError(f"Strategy '{c.strategy}' does not support online rollout")
        if c.parallel_mode in ("tp", "cp", "pp"):
            # responses are sampled by the serving scheduler from the training model itself; the sharded training forms of
            # these modes have no KV-cache forward
            raise ValueError(f"online rollouts sample from the training model, which parallel_mode '{c.parallel_mode}' cuts into "
                             "a training-only form; use none / ddp / fsdp / ep, or train offline on sampled data")
        from astrai_b200.inference.scheduler import InferenceScheduler
        from astrai_b200.tokenize import AutoTokenizer
        from astrai_b200.trainer.rollout import RolloutGenerator, RolloutRunner

        tokenizer = AutoTokenizer.from_pretrained(self._param_path)
        group = strategy_kwargs.get("group_size", 1)
        inner = getattr(ctx.model, "module", ctx.model)
        scheduler = InferenceScheduler(model=inner, tokenizer=tokenizer, max_batch_size=group * max(1, c.batch_per_device),
                                       max_seq_len=getattr(inner.config, "max_position_embeddings", None))
        generator = RolloutGenerator(scheduler=scheduler, tokenizer=tokenizer, max_tokens=c.rollout_max_tokens,
                                     group_size=group, temperature=c.rollout_temperature, top_k=c.rollout_top_k,
                                     top_p=c.rollout_top_p)
        ctx.strategy.set_rollout_runner(RolloutRunner(generator=generator, reward_model=c.reward_model_fn(),
                                                      rollout_interval=c.rollout_interval))
