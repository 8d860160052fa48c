"""Common behaviour of every config object: dict / JSON round trip.

Reference: ``astrai/config/base.py:10-38``.  ``to_dict`` keeps only values that
JSON can hold, so a config that mixes hyper-parameters with callables or
datasets (the training config) can still be written into checkpoint metadata.
"""

import dataclasses
import json
from pathlib import Path
from typing import Any, Dict, Union

from pydantic import ConfigDict
from pydantic.dataclasses import dataclass


def _jsonable(value) -> bool:
    try:
        json.dumps(value)
        return True
    except (TypeError, ValueError):
        return False


@dataclass(config=ConfigDict(use_attribute_docstrings=True))
class BaseConfig:
    def to_dict(self) -> Dict[str, Any]:
        out = {}
        for f in dataclasses.fields(self):
            value = getattr(self, f.name)
            if dataclasses.is_dataclass(value) and not isinstance(value, type):
                value = value.to_dict() if hasattr(value, "to_dict") else dataclasses.asdict(value)
            elif isinstance(value, tuple):
                value = list(value)
            if _jsonable(value):
                out[f.name] = value
        return out

    @classmethod
    def from_dict(cls, d: Dict[str, Any]):
        return cls(**d)

    @classmethod
    def from_file(cls, path: Union[str, Path]):
        with open(path, "r", encoding="utf-8") as fh:
            return cls.from_dict(json.load(fh))

    def to_file(self, path: Union[str, Path]):
        with open(path, "w", encoding="utf-8") as fh:
            json.dump(self.to_dict(), fh, indent=2, ensure_ascii=False)


def one_of(name: str, allowed):
    """Build a validator body that checks membership in *allowed*."""
    allowed = frozenset(allowed)

    def check(value):
        if value not in allowed:
            raise ValueError(f"{name} must be one of {sorted(allowed)}, got {value!r}")
        return value

    return check
