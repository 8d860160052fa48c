"""Shared CLI plumbing: YAML config files merged under explicit command-line options.

Precedence (lowest to highest): option default < YAML value < option given on the command line - the rule of the
reference's ``scripts/tools/train.py:76-98``.  YAML scalars that look like floats in YAML 1.2 but load as strings
with PyYAML (``1e-4``) are converted.
"""

from __future__ import annotations

import re
from typing import Any, Dict, Iterable, Optional

import click

_FLOAT = re.compile(r"^[+-]?(\d+\.?\d*|\.\d+)([eE][+-]?\d+)?$")


def _coerce(value: Any) -> Any:
    if isinstance(value, str) and _FLOAT.match(value.strip()) and any(c in value for c in ".eE"):
        try:
            return float(value)
        except ValueError:
            return value
    if isinstance(value, dict):
        return {k: _coerce(v) for k, v in value.items()}
    if isinstance(value, list):
        return [_coerce(v) for v in value]
    return value


def load_yaml(path: Optional[str]) -> Dict[str, Any]:
    if not path:
        return {}
    import yaml

    with open(path) as fh:
        data = yaml.safe_load(fh) or {}
    if not isinstance(data, dict):
        raise click.UsageError(f"{path}: the top level of a config file must be a mapping")
    return _coerce(data)


def flatten_sections(data: Dict[str, Any], sections: Iterable[str]) -> Dict[str, Any]:
    """Options may sit at the top level or inside any of the named sections (``model:``, ``training:`` ...)."""
    flat: Dict[str, Any] = {}
    for key, value in data.items():
        if key in sections and isinstance(value, dict):
            flat.update(value)
        elif key != "runtime":  # host-side section for container wrappers, not an option group
            flat[key] = value
    return flat


def merge_config(ctx: click.Context, params: Dict[str, Any], yaml_values: Dict[str, Any]) -> Dict[str, Any]:
    """Apply YAML values to every option the user did not pass explicitly; reject unknown keys."""
    known = {p.name for p in ctx.command.params}
    unknown = sorted(k for k in yaml_values if k.replace("-", "_") not in known)
    if unknown:
        raise click.UsageError(f"unknown option(s) in config file: {', '.join(unknown)}")
    merged = dict(params)
    for key, value in yaml_values.items():
        name = key.replace("-", "_")
        source = ctx.get_parameter_source(name)
        if source in (click.core.ParameterSource.DEFAULT, click.core.ParameterSource.DEFAULT_MAP, None):
            param = next(p for p in ctx.command.params if p.name == name)
            if param.multiple and not isinstance(value, (list, tuple)):
                value = [value]
            merged[name] = tuple(value) if param.multiple else value
    return merged


def torch_dtype(name: str):
    import torch

    table = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float16": torch.float16, "fp16": torch.float16,
             "float32": torch.float32, "fp32": torch.float32}
    if name not in table:
        raise click.BadParameter(f"unknown dtype {name!r}; choose from {sorted(table)}")
    return table[name]
