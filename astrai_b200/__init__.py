"""astrai_b200: a Blackwell-native (sm_100a) transformer training and serving framework.

The top level re-exports the same names a user of the reference imports from ``astrai``
(``astrai/__init__.py:51-93``), resolved lazily so that ``import astrai_b200`` stays cheap and never touches CUDA.
"""

from __future__ import annotations

import importlib
from typing import Any

__version__ = "0.2.0"

_EXPORTS = {
    # config
    "AutoRegressiveLMConfig": "astrai_b200.config", "BaseModelConfig": "astrai_b200.config",
    "ConfigFactory": "astrai_b200.config", "EncoderConfig": "astrai_b200.config", "PipelineConfig": "astrai_b200.config",
    "TrainConfig": "astrai_b200.config", "LoRAConfig": "astrai_b200.config",
    # data
    "BaseDataset": "astrai_b200.data", "DatasetFactory": "astrai_b200.data", "RDSampler": "astrai_b200.data",
    "Store": "astrai_b200.data", "StoreFactory": "astrai_b200.data",
    # core
    "BaseFactory": "astrai_b200.factory", "setup_logging": "astrai_b200.logging",
    # inference
    "InferenceEngine": "astrai_b200.inference", "get_app": "astrai_b200.inference", "run_server": "astrai_b200.inference",
    "sample": "astrai_b200.inference", "SamplingPipeline": "astrai_b200.inference",
    "ProtocolHandler": "astrai_b200.inference.network",
    # models
    "AutoModel": "astrai_b200.models", "AutoRegressiveLM": "astrai_b200.models", "EmbeddingEncoder": "astrai_b200.models",
    "inject_lora": "astrai_b200.models",
    # parallel
    "ExecutorFactory": "astrai_b200.parallel", "get_rank": "astrai_b200.parallel", "get_world_size": "astrai_b200.parallel",
    "only_on_rank": "astrai_b200.parallel", "spawn_parallel_fn": "astrai_b200.parallel",
    # data preparation / persistence
    "Pipeline": "astrai_b200.preprocessing", "filter_by_length": "astrai_b200.preprocessing",
    "Checkpoint": "astrai_b200.serialization", "AutoTokenizer": "astrai_b200.tokenize", "ChatTemplate": "astrai_b200.tokenize",
    # training
    "BaseScheduler": "astrai_b200.trainer", "BaseStrategy": "astrai_b200.trainer", "CallbackFactory": "astrai_b200.trainer",
    "SchedulerFactory": "astrai_b200.trainer", "StrategyFactory": "astrai_b200.trainer", "TrainCallback": "astrai_b200.trainer",
    "Trainer": "astrai_b200.trainer", "OptimizerFactory": "astrai_b200.optim",
}

__all__ = sorted(_EXPORTS)


def __getattr__(name: str) -> Any:
    target = _EXPORTS.get(name)
    if target is None:
        raise AttributeError(f"module 'astrai_b200' has no attribute {name!r}")
    value = getattr(importlib.import_module(target), name)
    globals()[name] = value
    return value


def __dir__():
    return sorted(list(globals()) + list(_EXPORTS))
