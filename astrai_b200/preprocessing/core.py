"""Helpers shared by the offline pipeline and the online JSONL transform (reference ``astrai/preprocessing/core.py``)."""

from __future__ import annotations

from itertools import chain
from typing import Dict, Iterator, List, Optional

import torch


def build_preprocessing_components(config, tokenizer_path: str):
    """(tokenizer, mask builder, position-id strategy) for a pipeline config."""
    from astrai_b200.preprocessing.builder import MaskBuilderFactory
    from astrai_b200.preprocessing.position_id import PositionIdStrategyFactory
    from astrai_b200.tokenize import AutoTokenizer

    return (AutoTokenizer.from_pretrained(tokenizer_path), MaskBuilderFactory.create("sectioned"),
            PositionIdStrategyFactory.create(config.output.position_ids_mode))


def primary_ids(result: dict) -> List[int]:
    """The first flat list of ints in a builder result (``sequence`` / ``chosen`` / ``prompts``)."""
    for v in result.values():
        if isinstance(v, list) and v and isinstance(v[0], int):
            return v
    return []


def infer_dtype(values: list) -> torch.dtype:
    """float32 for a column of floats (rewards), int32 for everything else."""
    return torch.float32 if values and isinstance(values[0], float) else torch.int32


def iter_raw_records(records: List[dict], mask_builder, config, tokenizer) -> Iterator[dict]:
    for item in records:
        result = mask_builder.build(item, config, tokenizer)
        if result is None:
            continue
        result.pop("domain", None)
        if primary_ids(result):
            yield result


def to_per_record_tensors(raw: Dict[str, list]) -> Dict[str, list]:
    """Per-record lists -> one tensor per record (nested lists -> list of tensors per record)."""
    out: Dict[str, list] = {}
    for key, column in raw.items():
        if column and isinstance(column[0], list):
            out[key] = [
                [torch.tensor(sub, dtype=infer_dtype(sub)) for sub in rec] if rec and isinstance(rec[0], list)
                else torch.tensor(rec, dtype=infer_dtype(rec))
                for rec in column
            ]
        else:
            out[key] = [torch.tensor(list(chain.from_iterable(column)), dtype=torch.int32)]
    return out


def build_position_ids(sequences: List[List[int]], strategy) -> Optional[List[int]]:
    return strategy.generate(sequences) or None
