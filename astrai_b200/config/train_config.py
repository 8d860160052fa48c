"""Training run configuration.

Reference: ``astrai/config/train_config.py:21-220``.  The reference accepts the
parallel modes ``none | ddp | fsdp``; this framework adds ``tp``, ``cp``, ``ep``
and the mesh sizes that go with them (the reference parses ``--tp_size`` and
then drops it, ``scripts/tools/train.py:513-550``).
"""

from dataclasses import field
from typing import Any, Callable, Dict, List, Optional

from pydantic import ConfigDict, field_validator, model_validator
from pydantic.dataclasses import dataclass

from astrai_b200.config.base import BaseConfig, one_of

TRAIN_TYPES = ("seq", "sft", "dpo", "grpo", "online_grpo", "online_dpo")
PARALLEL_MODES = ("none", "ddp", "fsdp", "tp", "cp", "ep", "pp")
BACKENDS = ("nccl", "gloo")
START_METHODS = ("spawn", "fork", "forkserver")
COMPILE_MODES = ("default", "reduce-overhead", "max-autotune")


@dataclass
class LoRAConfig:
    """Low-rank adapter settings (reference: ``astrai/model/components/lora.py:25-36``)."""

    r: int = 16
    alpha: int = 32
    target_modules: tuple = ("q_proj", "v_proj")


@dataclass(config=ConfigDict(arbitrary_types_allowed=True))
class TrainConfig(BaseConfig):
    model_fn: Callable[[], Any]
    strategy: str
    dataset: Any
    optimizer_fn: Callable[[Any], Any]
    scheduler_fn: Optional[Callable[[Any], Any]] = None
    optimizer_name: Optional[str] = None
    optimizer_hyperparameters: Dict[str, Any] = field(default_factory=dict)
    n_epoch: int = 1
    batch_per_device: int = 4
    grad_accum_steps: int = 1
    max_grad_norm: Optional[float] = 1.0
    gradient_checkpointing_modules: List[type] = field(default_factory=list)
    compile_mode: Optional[str] = None
    start_epoch: int = 0
    start_samples: int = 0
    ckpt_dir: str = "./checkpoint"
    ckpt_interval: int = 5000
    lora: Optional[LoRAConfig] = None
    metrics: List[str] = field(default_factory=lambda: ["loss", "lr", "grad_norm"])
    random_seed: int = 3407
    num_workers: int = 0
    prefetch_factor: Optional[int] = None
    persistent_workers: bool = False
    pin_memory: bool = False
    collate_fn: Optional[Callable[[List[Any]], Any]] = None
    nprocs: int = 1
    backend: str = "nccl"
    master_addr: str = "127.0.0.1"
    master_port: Optional[str] = "29500"
    parallel_mode: str = "none"
    tp_size: int = 1
    cp_size: int = 1
    ep_size: int = 1
    pp_size: int = 1
    start_method: str = "spawn"
    device_type: str = "cuda"
    val_dataset: Optional[Any] = None
    val_split: Optional[float] = None
    val_step: int = 1000
    neftune_alpha: float = 0.0
    moe_aux_loss_coef: float = 0.01
    rollout_interval: int = 512
    rollout_temperature: float = 0.7
    rollout_top_k: int = 0
    rollout_top_p: float = 0.9
    rollout_max_tokens: int = 1024
    reward_model_fn: Optional[Callable] = None
    executor_kwargs: Dict[str, Any] = field(default_factory=dict)
    strategy_kwargs: Dict[str, Any] = field(default_factory=dict)
    heartbeat_timeout_s: Optional[float] = None
    """If set (multi-rank runs), the trainer adds the ``heartbeat`` callback: a rank whose liveness entry in the
    process group's store is older than this many seconds is declared dead and the survivors stop between steps."""
    heartbeat_interval_s: float = 1.0

    @field_validator("strategy")
    def _c_strategy(cls, v):
        return one_of("strategy", TRAIN_TYPES)(v)

    @field_validator("parallel_mode")
    def _c_parallel(cls, v):
        return one_of("parallel_mode", PARALLEL_MODES)(v)

    @field_validator("backend")
    def _c_backend(cls, v):
        return one_of("backend", BACKENDS)(v)

    @field_validator("start_method")
    def _c_start(cls, v):
        return one_of("start_method", START_METHODS)(v)

    @field_validator("compile_mode")
    def _c_compile(cls, v):
        return v if v is None else one_of("compile_mode", COMPILE_MODES)(v)

    @field_validator(
        "n_epoch", "batch_per_device", "grad_accum_steps", "ckpt_interval", "val_step",
        "rollout_interval", "rollout_max_tokens", "tp_size", "cp_size", "ep_size", "pp_size",
    )
    def _c_positive(cls, v):
        if v <= 0:
            raise ValueError(f"must be positive, got {v}")
        return v

    @field_validator("rollout_temperature")
    def _c_temp(cls, v):
        if v <= 0:
            raise ValueError(f"must be positive, got {v}")
        return v

    @field_validator("rollout_top_p")
    def _c_top_p(cls, v):
        if not 0 < v <= 1:
            raise ValueError(f"rollout_top_p must be in (0, 1], got {v}")
        return v

    @field_validator("rollout_top_k", "num_workers", "neftune_alpha", "moe_aux_loss_coef")
    def _c_nonneg(cls, v):
        if v < 0:
            raise ValueError(f"must be non-negative, got {v}")
        return v

    @field_validator("max_grad_norm")
    def _c_clip(cls, v):
        if v is not None and v <= 0:
            raise ValueError(f"max_grad_norm must be positive or None, got {v}")
        return v

    @field_validator("val_split")
    def _c_split(cls, v):
        if v is not None and not 0 < v < 1:
            raise ValueError(f"val_split must be in (0, 1) or None, got {v}")
        return v

    @model_validator(mode="after")
    def _c_online(self):
        if self.strategy.startswith("online_") and self.reward_model_fn is None:
            raise ValueError(f"reward_model_fn is required for online RL strategy {self.strategy!r}")
        return self
