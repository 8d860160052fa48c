"""LoRA adapters on ``Linear`` layers: inject, merge, save, load.

Reference: ``astrai/model/components/lora.py:25-199`` - frozen base weight, ``A ~ randn / r``, ``B = 0``,
``scaling = alpha / r``; adapter files ``adapter_model.safetensors`` + ``adapter_config.json``; state-dict keys
``<module>.lora_A`` / ``<module>.lora_B``.
"""

from __future__ import annotations

import dataclasses
import logging
from pathlib import Path
from typing import Iterable, Optional, Set

import torch
import torch.nn as nn

from astrai_b200 import ops
from astrai_b200.config.train_config import LoRAConfig
from astrai_b200.models.layers import Linear
from astrai_b200.serialization import load_json, load_safetensors, save_json, save_safetensors

logger = logging.getLogger(__name__)

TARGET_MODULES_ATTN = {"q_proj", "k_proj", "v_proj", "o_proj"}
TARGET_MODULES_FFN = {"up", "gate", "down"}


class LoRALinear(nn.Module):
    def __init__(self, base: Linear, r: int = 16, alpha: int = 32):
        super().__init__()
        self.weight = base.weight
        self.weight.requires_grad_(False)
        self.bias = base.bias
        if self.bias is not None:
            self.bias.requires_grad_(False)
        self.r, self.scaling = r, alpha / r
        out_dim, in_dim = self.weight.shape
        opts = dict(device=self.weight.device, dtype=self.weight.dtype)
        self.lora_A = nn.Parameter(torch.randn(r, in_dim, **opts) / r)
        self.lora_B = nn.Parameter(torch.zeros(out_dim, r, **opts))
        self._merged = False

    def forward(self, x):
        y = ops.linear(x, self.weight, self.bias)
        if self._merged:
            return y
        return y + ops.linear(ops.linear(x, self.lora_A), self.lora_B) * self.scaling

    def merge(self):
        if self._merged:
            return
        with torch.no_grad():
            self.weight.add_((self.lora_B.float() @ self.lora_A.float()).to(self.weight.dtype) * self.scaling)
        self._merged = True
        del self.lora_A, self.lora_B


def _lora_layers(model: nn.Module):
    return [m for m in model.modules() if isinstance(m, LoRALinear)]


def inject_lora(model: nn.Module, r: int = 16, alpha: int = 32, target_modules: Optional[Iterable[str]] = None) -> LoRAConfig:
    """Wrap every ``Linear`` whose attribute name is in ``target_modules`` (default: the four attention projections)."""
    targets: Set[str] = set(target_modules) if target_modules is not None else set(TARGET_MODULES_ATTN)
    seen, count = set(), 0
    for name, module in list(model.named_modules()):
        if not isinstance(module, Linear):
            continue
        parent_name, _, leaf = name.rpartition(".")
        seen.add(leaf)
        if leaf in targets:
            parent = model.get_submodule(parent_name) if parent_name else model
            setattr(parent, leaf, LoRALinear(module, r=r, alpha=alpha))
            count += 1
    if count:
        logger.info("LoRA injected: %d layers (r=%d, alpha=%d)", count, r, alpha)
    else:
        logger.warning("No LoRA layers injected. Linear names present: %s; target_modules: %s", sorted(seen), sorted(targets))
    return LoRAConfig(r=r, alpha=alpha, target_modules=tuple(targets))


def merge_lora(model: nn.Module):
    layers = _lora_layers(model)
    for layer in layers:
        layer.merge()
    if layers:
        logger.info("Merged %d LoRA layers", len(layers))
    else:
        logger.warning("No LoRA layers to merge.")


def save_lora(model: nn.Module, save_dir: str, config: LoRAConfig):
    sd = {k: v for k, v in model.state_dict().items() if k.endswith((".lora_A", ".lora_B"))}
    if not sd:
        raise RuntimeError("No LoRA parameters found in model. The model may not have been injected or was already merged.")
    out = Path(save_dir)
    out.mkdir(parents=True, exist_ok=True)
    save_safetensors(sd, out / "adapter_model.safetensors")
    cfg = dataclasses.asdict(config)
    cfg["target_modules"] = list(cfg["target_modules"])
    save_json(cfg, out / "adapter_config.json")


def load_lora(model: nn.Module, load_dir: str) -> LoRAConfig:
    root = Path(load_dir)
    raw = load_json(root / "adapter_config.json")
    config = LoRAConfig(r=raw["r"], alpha=raw["alpha"], target_modules=tuple(raw["target_modules"]))
    if _lora_layers(model):
        logger.warning("Model already has LoRA layers; loading weights onto them without re-injecting.")
    else:
        inject_lora(model, r=config.r, alpha=config.alpha, target_modules=set(config.target_modules))
    weights = load_safetensors(root / "adapter_model.safetensors")
    try:
        missing, unexpected = model.load_state_dict(weights, strict=False)
    except RuntimeError as exc:
        if "size mismatch" in str(exc):
            raise RuntimeError(f"LoRA weight shapes do not match the model (adapter r={config.r}): {exc}") from exc
        raise
    if not _lora_layers(model):
        raise RuntimeError("No LoRA layers found after loading; check the adapter config.")
    absent = [k for k in missing if "lora" in k]
    if absent:
        raise RuntimeError(f"LoRA weight keys not found in the adapter file: {absent} (adapter r={config.r})")
    if unexpected:
        logger.warning("LoRA load: %d unexpected keys", len(unexpected))
    return config
