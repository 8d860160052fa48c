"""Token-shard files: one flat ``<key>.bin`` per key plus ``meta.json`` (shape, dtype, optional record offsets).

Format of the reference (``astrai/serialization/dataset.py:12-82``) so that its preprocessed data loads here.
"""

from __future__ import annotations

import json
import os
from typing import Any, Dict, List, Optional

import numpy as np
import torch
from torch import Tensor


def save_bin(file_path: str, tensor_group: Dict[str, List[Tensor]], record_keys: Optional[List[str]] = None):
    """Concatenate each key's tensors along dim 0 and dump them raw.  Keys named in ``record_keys`` also get
    cumulative per-record offsets so single records can be sliced back out."""
    os.makedirs(file_path, exist_ok=True)
    with_offsets = set(record_keys or ())
    meta: Dict[str, Any] = {}
    for key, parts in tensor_group.items():
        if parts and isinstance(parts[0], (list, tuple)):
            raise ValueError(f"Nested key '{key}' (List[List[Tensor]]) is not supported in bin format. Use JSONL storage instead.")
        flat = torch.cat(list(parts), dim=0)
        entry: Dict[str, Any] = {"shape": list(flat.shape), "dtype": str(flat.dtype).rsplit(".", 1)[-1]}
        if key in with_offsets:
            entry["offsets"] = [0] + np.cumsum([p.shape[0] for p in parts]).tolist()
        meta[key] = entry
        flat.cpu().numpy().tofile(os.path.join(file_path, f"{key}.bin"))
    with open(os.path.join(file_path, "meta.json"), "w") as fh:
        json.dump(meta, fh)


def _meta(file_path: str) -> dict:
    with open(os.path.join(file_path, "meta.json")) as fh:
        return json.load(fh)


def load_bin(file_path: str) -> Dict[str, List[Tensor]]:
    """Memory-map every key (copy-on-write) and wrap it as a single-segment list of tensors."""
    out: Dict[str, List[Tensor]] = {}
    for key, info in _meta(file_path).items():
        arr = np.memmap(os.path.join(file_path, f"{key}.bin"), dtype=info["dtype"], mode="c", shape=tuple(info["shape"]))
        out[key] = [torch.from_numpy(arr)]
    return out


def load_bin_offsets(file_path: str) -> Dict[str, List[int]]:
    return {k: v["offsets"] for k, v in _meta(file_path).items() if "offsets" in v}
