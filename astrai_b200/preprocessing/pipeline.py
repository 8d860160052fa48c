"""Offline preprocessing: JSON / JSONL -> tokenised, packed, sharded ``.bin`` stores.

Flow of the reference (``astrai/preprocessing/pipeline.py:50-277``): batches of records -> mask builder (batched
tokenisation, per-record retry when a batch fails) -> per-domain buckets -> when ``max_tokens_per_shard`` is reached:
doc-reset position ids -> packer -> tensors (per-key dtype overrides) -> continuous position ids -> writer.
"""

from __future__ import annotations

import json
import logging
import os
from collections import defaultdict
from itertools import chain
from typing import Dict, List, Optional

import torch

from astrai_b200.config import PipelineConfig
from astrai_b200.preprocessing.core import build_preprocessing_components, primary_ids
from astrai_b200.preprocessing.packing import PackingStrategyFactory
from astrai_b200.preprocessing.writer import StoreWriterFactory

logger = logging.getLogger(__name__)

DTYPES = {n: getattr(torch, n) for n in ("bool", "uint8", "int8", "int16", "int32", "int64", "float16", "float32", "float64")}


def filter_by_length(text: str, min_len: int = 50, max_len: int = 2_000_000) -> bool:
    return min_len <= len(text) <= max_len


class Pipeline:
    def __init__(self, config: PipelineConfig, input_paths: List[str], output_dir: str, tokenizer_path: str):
        os.makedirs(output_dir, exist_ok=True)
        self.config, self.paths, self.output_dir, self.tokenizer_path = config, list(input_paths), output_dir, tokenizer_path
        self.tokenizer, self.mask_builder, self._position_id = build_preprocessing_components(config, tokenizer_path)
        self._packer = PackingStrategyFactory.create(config.preprocessing.packing_strategy)
        self._writer = StoreWriterFactory.create(config.output.storage_format)

    def transform(self, item: dict) -> Optional[dict]:
        return self.mask_builder.build(item, self.config, self.tokenizer)

    def transform_batch(self, items: List[dict]) -> List[Optional[dict]]:
        return self.mask_builder.build_batch(items, self.config, self.tokenizer)

    # -- input ---------------------------------------------------------------------------------------------------------
    def _records(self):
        for path in self.paths:
            with open(path, "r", encoding="utf-8") as fh:
                if path.endswith(".json"):
                    data = json.load(fh)
                    yield from (data if isinstance(data, list) else [data])
                else:
                    for n, line in enumerate(fh, 1):
                        if not line.strip():
                            continue
                        try:
                            rec = json.loads(line)
                        except json.JSONDecodeError:
                            logger.warning("%s:%d is not valid JSON, skipped", path, n)
                            continue
                        if isinstance(rec, dict):
                            yield rec

    def _batches(self, size: int):
        batch = []
        for rec in self._records():
            batch.append(rec)
            if len(batch) >= max(1, size):
                yield batch
                batch = []
        if batch:
            yield batch

    def _safe_transform(self, items):
        try:
            return self.transform_batch(items)
        except Exception:
            logger.warning("Failed to process batch, retrying records individually", exc_info=True)
        out = []
        for item in items:
            try:
                out.append(self.transform(item))
            except Exception:
                logger.warning("Failed to process item, skipping", exc_info=True)
                out.append(None)
        return out

    # -- main loop -------------------------------------------------------------------------------------------------------
    def run(self):
        pp, limit = self.config.preprocessing, self.config.output.max_tokens_per_shard
        buckets: dict = defaultdict(lambda: defaultdict(list))
        shard_idx: Dict[str, int] = defaultdict(int)
        tokens = kept = 0
        for items in self._batches(pp.batch_size):
            done = False
            for result in self._safe_transform(items):
                if pp.max_items and kept >= pp.max_items:
                    done = True
                    break
                if result is None:
                    continue
                domain = result.pop("domain", "__default__")
                ids = primary_ids(result)
                if not ids:
                    continue
                bucket = buckets[domain]
                for key in bucket:  # keep columns aligned when this record lacks a key seen before
                    if key not in result:
                        bucket[key].append([0] * len(ids))
                for key, val in result.items():
                    bucket[key].append(val)
                kept += 1
                tokens += len(ids)
                if tokens >= limit:
                    self._flush(buckets, shard_idx)
                    buckets.clear()
                    tokens = 0
            if done:
                break
        if tokens > 0:
            self._flush(buckets, shard_idx)
        return kept

    def _flush(self, buckets, shard_idx):
        pp, mode = self.config.preprocessing, self.config.output.position_ids_mode
        for domain, keys in buckets.items():
            keys = dict(keys)
            docs = keys.get("sequence", [])
            if mode == "doc_reset" and docs:  # must enter the packer so bins concatenate per-document ranges
                keys["position_ids"] = [list(range(len(d))) for d in docs]
            keys = self._packer.apply(keys, pp.max_packed_len, pp.truncation_mode)
            tensors = self._to_tensors(keys)
            if mode == "continuous" and keys.get("sequence"):
                pos = self._position_id.generate(keys["sequence"])
                if pos:
                    tensors["position_ids"] = [torch.tensor(pos, dtype=torch.int32)]
            idx = shard_idx[domain]
            # multi-output records (preference pairs ...) are read back one by one: keep their boundaries in the shard
            record_keys = list(tensors) if getattr(self.config.input, "sources", None) else None
            self._writer.save(self.output_dir, domain, idx, tensors, record_keys=record_keys)
            shard_idx[domain] = idx + 1
            first = "sequence" if "sequence" in tensors else next(iter(tensors))
            logger.info("saved %s/shard_%04d (%d records)", domain, idx, len(tensors[first]))

    def _to_tensors(self, keys: Dict[str, list]) -> Dict[str, List[torch.Tensor]]:
        """Columns of id lists as tensors.  Per-record columns give one tensor per record; a record that is itself a list
        of lists (a group of responses) is flattened for ``bin`` shards, as the reference does, and kept as a list of
        tensors for ``jsonl`` shards, which can store the boundaries.  The dtype is the configured one, else float32
        for columns that hold floats (rewards) and int32 for the rest."""
        keep_nested = self.config.output.storage_format == "jsonl"
        out: Dict[str, List[torch.Tensor]] = {}
        for key, column in keys.items():
            name = self.config.output.dtype.get(key)
            if name is not None:
                dtype = DTYPES.get(name, torch.int32)
            else:
                probe = column
                while probe and isinstance(probe[0], list):
                    probe = probe[0]
                dtype = torch.float32 if (probe and isinstance(probe[0], float)) else torch.int32
            if column and isinstance(column[0], list):
                recs = []
                for rec in column:
                    if rec and isinstance(rec[0], list):
                        recs.append([torch.tensor(r, dtype=dtype) for r in rec] if keep_nested
                                    else torch.tensor(list(chain.from_iterable(rec)), dtype=dtype))
                    else:
                        recs.append(torch.tensor(rec, dtype=dtype))
                out[key] = recs
            else:
                out[key] = [torch.tensor(list(chain.from_iterable(column)), dtype=dtype)]
        return out
