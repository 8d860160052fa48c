"""Checkpoint and model-directory I/O.

On-disk layout is the reference's (``astrai/serialization/checkpoint.py:152-209``):
``meta.json`` (epoch, consumed_samples, timestamp, + caller metadata), ``config.json`` (model config),
``model.safetensors`` (full, unsharded weights), one ``<name>.pt`` per extra object (optimizer, scheduler).
Additions: a checkpoint is written into ``<dir>.tmp`` and renamed into place, and ``meta.json`` is written last,
so a directory that has ``meta.json`` is complete; rank-0-load-then-broadcast is available on every loader.
"""

from __future__ import annotations

import io
import json
import os
import shutil
import time
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Callable, Dict, Optional, Union

import safetensors.torch as st
import torch
import torch.distributed as dist

META_FILE, CONFIG_FILE, WEIGHTS_FILE = "meta.json", "config.json", "model.safetensors"
INDEX_FILE = "model.safetensors.index.json"
PathLike = Union[str, Path]


def _rank() -> int:
    return dist.get_rank() if dist.is_available() and dist.is_initialized() else 0


def _distributed() -> bool:
    return dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1


def _object_from_rank0(loader: Callable[[], Any], broadcast: bool):
    if not (broadcast and _distributed()):
        return loader()
    box = [loader() if _rank() == 0 else None]
    dist.broadcast_object_list(box, src=0)
    return box[0]


def save_json(data: dict, path: PathLike):
    Path(path).write_text(json.dumps(data, indent=2))


def load_json(path: PathLike, broadcast: bool = False) -> dict:
    return _object_from_rank0(lambda: json.loads(Path(path).read_text()), broadcast)


def save_safetensors(state_dict: dict, path: PathLike):
    """Every tensor is written from storage of its own: a device tensor is copied by the transfer, a host tensor is cloned
    (views of one flat buffer, or one tensor under two names, would otherwise be refused by the file format)."""
    def own(t):
        t = t.detach()
        return t.contiguous().cpu() if t.device.type != "cpu" else t.contiguous().clone()

    st.save_file({k: own(v) for k, v in state_dict.items()}, str(path))


def load_safetensors(path: PathLike, broadcast: bool = False) -> dict:
    return _object_from_rank0(lambda: st.load_file(str(path)), broadcast)


def save_torch(obj: Any, path: PathLike):
    torch.save(obj, str(path))


def load_torch(path: PathLike, broadcast: bool = False) -> Any:
    if not (broadcast and _distributed()):
        return torch.load(str(path), map_location="cpu", weights_only=False)
    if _rank() == 0:
        blob = torch.frombuffer(bytearray(Path(path).read_bytes()), dtype=torch.uint8)
        size = torch.tensor([blob.numel()], dtype=torch.long)
    else:
        size = torch.zeros(1, dtype=torch.long)
    dist.broadcast(size, src=0)
    if _rank() != 0:
        blob = torch.empty(int(size), dtype=torch.uint8)
    dist.broadcast(blob, src=0)
    return torch.load(io.BytesIO(blob.numpy().tobytes()), map_location="cpu", weights_only=False)


def load_state_dict(path: PathLike, broadcast: bool = False) -> dict:
    """Read one safetensors file; with ``broadcast`` rank 0 reads and sends tensor by tensor (CPU)."""
    if not (broadcast and _distributed()):
        return load_safetensors(path)
    sd = load_safetensors(path) if _rank() == 0 else {}
    specs = [[(k, tuple(v.shape), v.dtype) for k, v in sorted(sd.items())]]
    dist.broadcast_object_list(specs, src=0)
    for key, shape, dtype in specs[0]:
        t = sd[key].contiguous().cpu() if _rank() == 0 else torch.empty(shape, dtype=dtype)
        dist.broadcast(t, src=0)
        sd[key] = t
    return sd


def save_model(config: dict, state_dict: dict, save_directory: PathLike):
    out = Path(save_directory)
    out.mkdir(parents=True, exist_ok=True)
    save_json(config, out / CONFIG_FILE)
    save_safetensors(state_dict, out / WEIGHTS_FILE)


def load_model_config(save_directory: PathLike) -> dict:
    return load_json(Path(save_directory) / CONFIG_FILE)


def load_model_weights(save_directory: PathLike) -> dict:
    """``model.safetensors`` or the shards listed by ``model.safetensors.index.json``."""
    root = Path(save_directory)
    if (root / WEIGHTS_FILE).exists():
        return load_state_dict(root / WEIGHTS_FILE)
    if (root / INDEX_FILE).exists():
        merged: Dict[str, torch.Tensor] = {}
        for shard in sorted(set(load_json(root / INDEX_FILE).get("weight_map", {}).values())):
            merged.update(load_state_dict(root / shard))
        return merged
    raise FileNotFoundError(f"No model weights found in {save_directory}")


REQUIRED_FOR_RESUME = (META_FILE, CONFIG_FILE, WEIGHTS_FILE, "optimizer.pt", "scheduler.pt")


def is_complete(ckpt_dir: PathLike, need=None) -> bool:
    """True when a run can resume from ``ckpt_dir``: every file it needs exists and is non-empty.

    A checkpoint written here lists its files in ``meta.json`` (``files``): those must all be there, the optimizer state
    among them (a run without a learning-rate scheduler writes no ``scheduler.pt`` and is complete without it).  A
    directory without that list is held to the fixed set of the reference's tooling
    (``scripts/docker/lib/train-common.sh:25-66``: meta, config, weights, optimizer, scheduler)."""
    root = Path(ckpt_dir)
    if need is None:
        need = REQUIRED_FOR_RESUME
        meta_path = root / META_FILE
        if meta_path.is_file() and meta_path.stat().st_size > 0:
            try:
                listed = json.loads(meta_path.read_text(encoding="utf-8")).get("files")
            except (OSError, ValueError, AttributeError):
                listed = None  # not this writer's file: the fixed set decides
            if isinstance(listed, list) and listed:
                if "optimizer.pt" not in listed:
                    return False
                need = [META_FILE, *listed]
    return all((root / n).is_file() and (root / n).stat().st_size > 0 for n in need)


def latest_complete(ckpt_root: PathLike) -> Optional[Path]:
    """Newest ``epoch_*_step_*`` directory under ``ckpt_root`` that :func:`is_complete`."""
    root = Path(ckpt_root)
    if not root.is_dir():
        return None

    def step_of(p: Path):
        parts = p.name.split("_")
        try:
            return int(parts[1]), int(parts[3])
        except (IndexError, ValueError):
            return (-1, -1)

    for cand in sorted((p for p in root.iterdir() if p.is_dir() and p.name.startswith("epoch_")), key=step_of, reverse=True):
        if is_complete(cand):
            return cand
    return None


@dataclass
class Checkpoint:
    state_dict: Dict[str, Any] = field(default_factory=dict)
    epoch: int = 0
    consumed_samples: int = 0
    extra: Dict[str, Any] = field(default_factory=dict)
    meta: Dict[str, Any] = field(default_factory=dict)
    config: Dict[str, Any] = field(default_factory=dict)

    def save(self, save_dir: PathLike):
        final = Path(save_dir)
        final.parent.mkdir(parents=True, exist_ok=True)
        tmp = final.with_name(final.name + ".tmp")
        if tmp.exists():
            shutil.rmtree(tmp)
        tmp.mkdir(parents=True)
        save_json(self.config, tmp / CONFIG_FILE)
        save_safetensors(self.state_dict, tmp / WEIGHTS_FILE)
        for name, obj in self.extra.items():
            save_torch(obj, tmp / f"{name}.pt")
        written = sorted(p.name for p in tmp.iterdir())
        meta = {"epoch": self.epoch, "consumed_samples": self.consumed_samples,
                "timestamp": time.strftime("%Y-%m-%dT%H:%M:%S"), **self.meta, "files": written}
        save_json(meta, tmp / META_FILE)  # last: its presence marks a complete checkpoint
        if final.exists():
            # keep files other writers placed there (metric.jsonl), replace ours
            for item in tmp.iterdir():
                os.replace(item, final / item.name)
            tmp.rmdir()
        else:
            os.replace(tmp, final)

    @classmethod
    def load(cls, save_dir: PathLike, broadcast: bool = False) -> "Checkpoint":
        root = Path(save_dir)
        meta = load_json(root / META_FILE, broadcast)
        config = load_json(root / CONFIG_FILE, broadcast)
        sd = load_state_dict(root / WEIGHTS_FILE, broadcast=broadcast)
        # which extra files exist is rank 0's knowledge too: the other ranks may not see the directory at all
        names = _object_from_rank0(lambda: sorted(f.name for f in root.glob("*.pt")), broadcast)
        extra = {Path(n).stem: load_torch(root / n, broadcast=broadcast) for n in names}
        return cls(sd, meta.get("epoch", 0), meta.get("consumed_samples", 0), extra, meta, config)

    @classmethod
    def load_any(cls, save_dir: PathLike, broadcast: bool = False) -> Optional["Checkpoint"]:
        """A training checkpoint, a plain model directory, or a sharded HF-style directory; else None."""
        root = Path(save_dir)
        if (root / META_FILE).exists():
            return cls.load(root, broadcast=broadcast)
        if (root / WEIGHTS_FILE).exists() or (root / INDEX_FILE).exists():
            config = load_json(root / CONFIG_FILE, broadcast) if (root / CONFIG_FILE).exists() else {}
            return cls(state_dict=load_model_weights(root), config=config)
        return None
