from astrai_b200.config.base import BaseConfig
from astrai_b200.config.model_config import (
    AutoRegressiveLMConfig,
    BaseModelConfig,
    ConfigFactory,
    EncoderConfig,
)
from astrai_b200.config.preprocess_config import (
    InputConfig,
    OutputConfig,
    PipelineConfig,
    ProcessingConfig,
)
from astrai_b200.config.train_config import LoRAConfig, TrainConfig

__all__ = [
    "AutoRegressiveLMConfig", "BaseConfig", "BaseModelConfig", "ConfigFactory", "EncoderConfig",
    "InputConfig", "LoRAConfig", "OutputConfig", "PipelineConfig", "ProcessingConfig", "TrainConfig",
]
