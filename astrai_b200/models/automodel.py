"""Model registry and the load / save entry points shared by all model families.

``AutoModel.from_pretrained`` reads ``config.json`` (+ ``model.safetensors`` or a sharded index), recognises
HuggingFace LLaMA-layout checkpoints and converts them, and can skip random initialisation while it builds the
module tree (reference: ``astrai/model/automodel.py:24-130``).
"""

from __future__ import annotations

import contextlib
from pathlib import Path
from typing import Union

import torch.nn as nn

from astrai_b200.config.model_config import BaseModelConfig, ConfigFactory
from astrai_b200.factory import BaseFactory
from astrai_b200.serialization import (
    HF_MODEL_TYPES, adapt_config, convert_hf_weights, load_model_config, load_model_weights,
    looks_like_hf_state_dict, save_model,
)

_INIT_FNS = ("xavier_normal_", "xavier_uniform_", "kaiming_normal_", "kaiming_uniform_", "zeros_", "ones_",
             "constant_", "normal_", "uniform_", "trunc_normal_")


@contextlib.contextmanager
def skip_init(enabled: bool = True):
    """Turn ``torch.nn.init.*`` into no-ops: weights are about to be overwritten by a checkpoint."""
    if not enabled:
        yield
        return
    saved = {n: getattr(nn.init, n) for n in _INIT_FNS if hasattr(nn.init, n)}
    for n in saved:
        setattr(nn.init, n, lambda tensor, *a, **k: tensor)
    try:
        yield
    finally:
        for n, fn in saved.items():
            setattr(nn.init, n, fn)


class ModelFactory(BaseFactory[nn.Module]):
    """``model_type`` -> model class."""


class AutoModel(nn.Module):
    def __init__(self, config: BaseModelConfig):
        super().__init__()
        self.config = config

    @classmethod
    def from_pretrained(cls, path: Union[str, Path], disable_random_init: bool = True, strict: bool = True,
                        weights_format: str = "auto") -> nn.Module:
        if weights_format not in ("auto", "astrai", "hf"):
            raise ValueError(f"weights_format must be one of 'auto', 'astrai', 'hf', got {weights_format!r}")
        root = Path(path)
        if not (root / "config.json").exists():
            raise FileNotFoundError(f"Config file not found: {root / 'config.json'}")
        raw = load_model_config(root)
        hf_config = weights_format == "hf" or (weights_format == "auto" and raw.get("model_type") in HF_MODEL_TYPES)
        if hf_config:
            raw = adapt_config(raw) if raw.get("model_type") in HF_MODEL_TYPES else raw
        config = ConfigFactory.load(raw)
        model_cls = ModelFactory.get_component_class(config.model_type or ConfigFactory.DEFAULT_TYPE)
        with skip_init(disable_random_init):
            model = model_cls(config)
        if (root / "model.safetensors").exists() or (root / "model.safetensors.index.json").exists():
            sd = load_model_weights(root)
            if hf_config or (weights_format == "auto" and looks_like_hf_state_dict(sd)):
                sd = convert_hf_weights(sd, config)
            model.load_state_dict(sd, strict=strict)
        return model

    def save_pretrained(self, save_directory: Union[str, Path]):
        save_model(config=self.config.to_dict(), state_dict=self.state_dict(), save_directory=save_directory)
