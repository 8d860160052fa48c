"""Shard writers (reference ``astrai/preprocessing/writer.py:23-56``): ``<out>/<domain>/shard_%04d/``."""

from __future__ import annotations

import logging
import os
import shutil
from typing import Dict, List, Optional

import torch

from astrai_b200.factory import BaseFactory
from astrai_b200.serialization import save_bin

logger = logging.getLogger(__name__)


class StoreWriter:
    def save(self, output_dir: str, domain: str, shard_idx: int, tensors: Dict[str, List[torch.Tensor]],
             record_keys: Optional[List[str]] = None) -> None:
        """``record_keys``: columns whose per-record boundaries must survive (preference pairs, response groups)."""
        raise NotImplementedError


class StoreWriterFactory(BaseFactory["StoreWriter"]):
    pass


@StoreWriterFactory.register("bin")
class BinWriter(StoreWriter):
    def save(self, output_dir, domain, shard_idx, tensors, record_keys=None):
        path = os.path.join(output_dir, domain, f"shard_{shard_idx:04d}")
        try:
            save_bin(path, tensors, record_keys=record_keys)
        except Exception:
            shutil.rmtree(path, ignore_errors=True)  # never leave a half-written shard behind
            logger.error("Failed to write shard %s/shard_%04d, cleaned up partial output", domain, shard_idx, exc_info=True)
            raise


@StoreWriterFactory.register("jsonl")
class JsonlWriter(StoreWriter):
    """One JSON object per record with plain lists; readable by ``JsonlStore`` in processor mode."""

    @staticmethod
    def _plain(value):
        return [t.tolist() for t in value] if isinstance(value, (list, tuple)) else value.tolist()

    def save(self, output_dir, domain, shard_idx, tensors, record_keys=None):
        import json

        os.makedirs(os.path.join(output_dir, domain), exist_ok=True)
        path = os.path.join(output_dir, domain, f"shard_{shard_idx:04d}.jsonl")
        n = max(len(v) for v in tensors.values())
        with open(path, "w", encoding="utf-8") as fh:
            for i in range(n):
                row = {k: (self._plain(v[i]) if i < len(v) else None) for k, v in tensors.items()}
                fh.write(json.dumps(row) + "\n")
