from astrai_b200.trainer.schedule import BaseScheduler, CosineScheduler, SchedulerFactory, SGDRScheduler, WSDScheduler
from astrai_b200.trainer.strategy import (
    BaseStrategy, DPOStrategy, GRPOStrategy, SEQStrategy, SFTStrategy, StrategyFactory,
)
from astrai_b200.trainer.train_callback import (
    CallbackFactory, CheckpointCallback, GradientCheckpointingCallback, GradientClippingCallback, MetricCallback,
    ProgressBarCallback, TrainCallback,
)
from astrai_b200.trainer.train_context import TrainContext, TrainContextBuilder
from astrai_b200.trainer.trainer import Trainer

__all__ = [
    "BaseScheduler", "BaseStrategy", "CallbackFactory", "CheckpointCallback", "CosineScheduler", "DPOStrategy",
    "GRPOStrategy", "GradientCheckpointingCallback", "GradientClippingCallback", "MetricCallback",
    "ProgressBarCallback", "SEQStrategy", "SFTStrategy", "SGDRScheduler", "SchedulerFactory", "StrategyFactory",
    "TrainCallback", "TrainContext", "TrainContextBuilder", "Trainer", "WSDScheduler",
]
