"""Declarative description of the JSONL -> token-shard preprocessing pipeline.

Reference: ``astrai/config/preprocess_config.py:22-152``.
"""

from dataclasses import field
from typing import Dict, List, Optional

from pydantic import field_validator
from pydantic.dataclasses import dataclass

from astrai_b200.config.base import BaseConfig, one_of

PACKING_STRATEGIES = ("simple", "bfd", "bfd_split")
TRUNCATION_MODES = ("keep_start", "keep_end")
STORAGE_FORMATS = ("bin", "jsonl")
POSITION_ID_MODES = ("none", "doc_reset", "continuous")


def _positive(v):
    if v <= 0:
        raise ValueError(f"must be positive, got {v}")
    return v


@dataclass
class InputConfig(BaseConfig):
    """Either ``sections`` (one output stream) or ``sources`` (named streams, DPO/GRPO)."""

    sections: Optional[List[Dict]] = None
    sources: Optional[Dict[str, Dict]] = None


@dataclass
class ProcessingConfig(BaseConfig):
    max_seq_len: int = 2048
    min_chars: int = 50
    max_chars: int = 2_000_000
    max_items: Optional[int] = None
    batch_size: int = 256
    packing_strategy: str = "simple"
    max_packed_len: int = 8192
    truncation_mode: str = "keep_start"

    @field_validator("packing_strategy")
    def _check_pack(cls, v):
        return one_of("packing_strategy", PACKING_STRATEGIES)(v)

    @field_validator("truncation_mode")
    def _check_trunc(cls, v):
        return one_of("truncation_mode", TRUNCATION_MODES)(v)

    @field_validator("max_seq_len", "batch_size", "max_packed_len")
    def _check_pos(cls, v):
        return _positive(v)

    @field_validator("min_chars")
    def _check_min_chars(cls, v):
        if v < 0:
            raise ValueError(f"min_chars must be non-negative, got {v}")
        return v


@dataclass
class OutputConfig(BaseConfig):
    domain_key: Optional[str] = None
    storage_format: str = "bin"
    max_tokens_per_shard: int = 100_000_000
    dtype: Dict[str, str] = field(default_factory=dict)
    position_ids_mode: str = "doc_reset"

    @field_validator("storage_format")
    def _check_fmt(cls, v):
        return one_of("storage_format", STORAGE_FORMATS)(v)

    @field_validator("position_ids_mode")
    def _check_pos_mode(cls, v):
        return one_of("position_ids_mode", POSITION_ID_MODES)(v)


@dataclass
class PipelineConfig(BaseConfig):
    version: int = 1
    input: InputConfig = field(default_factory=InputConfig)
    mask: Dict[str, str] = field(default_factory=dict)
    mask_default: str = "mask"
    preprocessing: ProcessingConfig = field(default_factory=ProcessingConfig)
    output: OutputConfig = field(default_factory=OutputConfig)
