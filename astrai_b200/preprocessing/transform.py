"""Online tokenisation of raw JSONL records into per-record tensors (reference ``astrai/preprocessing/transform.py``)."""

from __future__ import annotations

import json
from pathlib import Path
from typing import Dict, List

import torch

from astrai_b200.config import PipelineConfig
from astrai_b200.preprocessing.core import (
    build_position_ids, build_preprocessing_components, iter_raw_records, primary_ids, to_per_record_tensors,
)


class TokenizeTransform:
    def __init__(self, config: PipelineConfig, tokenizer_path: str):
        self.config = config
        self.tokenizer, self.mask_builder, self.position_strategy = build_preprocessing_components(config, tokenizer_path)

    @classmethod
    def from_config_file(cls, config_path: str) -> "TokenizeTransform":
        """``dataset_config.json``: a pipeline config plus optional ``tokenizer_path`` (default: the file's directory)."""
        raw = json.loads(Path(config_path).read_text(encoding="utf-8"))
        tokenizer_path = raw.pop("tokenizer_path", None) or str(Path(config_path).parent)
        return cls(PipelineConfig.from_dict(raw), tokenizer_path)

    def apply(self, records: List[dict]) -> Dict[str, list]:
        columns: Dict[str, list] = {}
        docs: List[List[int]] = []
        for result in iter_raw_records(records, self.mask_builder, self.config, self.tokenizer):
            main = primary_ids(result)
            if main:
                docs.append(main)
            for key, ids in result.items():
                columns.setdefault(key, []).append(ids)
        tensors = to_per_record_tensors(columns)
        pos = build_position_ids(docs, self.position_strategy)
        if pos is not None:
            tensors["position_ids"] = [torch.tensor(pos, dtype=torch.int32)]
        return tensors
