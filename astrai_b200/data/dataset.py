"""Datasets: thin bindings of a :class:`Store` to the tensors each training strategy expects.

Reference: ``astrai/dataset/dataset.py:73-535``.  ``seq``: (window, window shifted by one); ``sft``: adds
``position_ids`` and the shifted ``loss_mask``; ``dpo`` / ``grpo``: one record per sample, padded by their collate
functions (prompts are LEFT-padded for GRPO).  ``SyntheticTokenDataset`` generates packed uniform token ids for
benchmarks and tests.
"""

from __future__ import annotations

from functools import partial
from pathlib import Path
from typing import Any, Callable, Dict, List, Optional

import torch
from torch import Tensor
from torch.utils.data import Dataset

from astrai_b200.data.storage import Store, StoreFactory, detect_format
from astrai_b200.factory import BaseFactory

DEFAULT_MESSAGES_CONFIG = {
    "version": 1,
    "input": {"sections": [{"field": "messages", "action": "$role", "template": True}]},
    "mask": {"system": "mask", "user": "mask", "assistant": "train"},
    "mask_default": "mask",
    "output": {"position_ids_mode": "doc_reset"},
}


# ------------------------------------------------------------------------------------------- DPO record helpers
def _as_messages(value) -> list:
    if isinstance(value, list):
        return value
    return [{"role": "user", "content": value if isinstance(value, str) else str(value)}]


def _as_text(value) -> Optional[str]:
    if isinstance(value, str):
        return value
    if isinstance(value, list):
        return "".join(m.get("content", "") for m in value if isinstance(m, dict))
    return None


def dpo_tokenize(record: dict, tokenizer, max_len: int = 2048) -> Optional[dict]:
    """Chat-template a preference pair; loss masks cover only the completion tokens."""
    prompt = record.get("prompt") or record.get("input")
    chosen, rejected = _as_text(record.get("chosen")), _as_text(record.get("rejected"))
    if prompt is None or chosen is None or rejected is None:
        return None
    msgs = _as_messages(prompt)
    n_prompt = min(len(tokenizer.apply_chat_template(msgs, tokenize=True, add_generation_prompt=True)), max_len)
    out = {}
    for name, text in (("chosen", chosen), ("rejected", rejected)):
        ids = tokenizer.apply_chat_template(msgs + [{"role": "assistant", "content": text}], tokenize=True,
                                            add_generation_prompt=False)[:max_len]
        out[name] = ids
        out[name + "_mask"] = ([0] * n_prompt + [1] * max(0, len(ids) - n_prompt))[:max_len]
    return out


def dpo_processor(record: dict, tokenizer, max_len: int = 2048) -> Dict[str, Tensor]:
    res = dpo_tokenize(record, tokenizer, max_len=max_len)
    if res is None:
        raise ValueError(f"Malformed DPO record: {list(record.keys())}")
    return {
        "chosen": torch.tensor(res["chosen"], dtype=torch.int32),
        "rejected": torch.tensor(res["rejected"], dtype=torch.int32),
        "chosen_mask": torch.tensor(res["chosen_mask"], dtype=torch.bool),
        "rejected_mask": torch.tensor(res["rejected_mask"], dtype=torch.bool),
    }


def pretokenized_processor(record: dict) -> Dict[str, Any]:
    """A record of id lists (as the pipeline's JSONL writer stores them) as tensors; nested lists stay lists of tensors."""
    out: Dict[str, Any] = {}
    for key, value in record.items():
        if not isinstance(value, list):
            continue
        if value and isinstance(value[0], list):
            out[key] = [torch.tensor(v) for v in value]
        else:
            out[key] = torch.tensor(value)
    return out


def dpo_collate_fn(batch: List[Dict[str, Tensor]]) -> Dict[str, Tensor]:
    """Right-pad chosen / rejected (and masks) to the longest sequence of the batch; pad id 0."""
    width = max(max(b["chosen"].numel(), b["rejected"].numel()) for b in batch)
    out = {
        "chosen": torch.zeros(len(batch), width, dtype=torch.long),
        "rejected": torch.zeros(len(batch), width, dtype=torch.long),
        "chosen_mask": torch.zeros(len(batch), width, dtype=torch.bool),
        "rejected_mask": torch.zeros(len(batch), width, dtype=torch.bool),
    }
    for i, b in enumerate(batch):
        for k in out:
            out[k][i, : b[k].numel()] = b[k]
    return out


def grpo_collate_fn(batch: List[Dict[str, Tensor]]) -> Dict[str, Tensor]:
    """prompts ``[B,P]`` left-padded (+ ``prompt_mask``), responses / masks ``[B,G,R]`` right-padded, rewards ``[B,G]``."""
    n, g = len(batch), len(batch[0]["responses"])
    p_max = max(b["prompts"].numel() for b in batch)
    r_max = max(r.numel() for b in batch for r in b["responses"])
    prompts = torch.zeros(n, p_max, dtype=torch.long)
    prompt_mask = torch.zeros(n, p_max, dtype=torch.bool)
    responses = torch.zeros(n, g, r_max, dtype=torch.long)
    masks = torch.zeros(n, g, r_max, dtype=torch.bool)
    rewards = torch.zeros(n, g, dtype=torch.float32)
    for i, b in enumerate(batch):
        plen = b["prompts"].numel()
        prompts[i, p_max - plen:] = b["prompts"]
        prompt_mask[i, p_max - plen:] = True
        rewards[i, : b["rewards"].numel()] = b["rewards"]
        for j, r in enumerate(b["responses"][:g]):
            responses[i, j, : r.numel()] = r
            if j < len(b["masks"]):
                masks[i, j, : r.numel()] = b["masks"][j]
    return {"prompts": prompts, "prompt_mask": prompt_mask, "responses": responses, "masks": masks, "rewards": rewards}


# ------------------------------------------------------------------------------------------- datasets
def validate_keys(store: Store, required: List[str]) -> None:
    """``KeyError`` naming the keys of ``required`` that ``store`` lacks (``astrai/dataset/dataset.py:260-270``)."""
    missing = [k for k in required if k not in set(store.keys)]
    if missing:
        raise KeyError(f"Store at {getattr(store, '_load_path', '?')} is missing required keys {missing}; "
                       f"available keys are {sorted(store.keys)}.")


class BaseDataset(Dataset):
    required_keys: List[str] = []

    def __init__(self, store: Store):
        self.store = store
        validate_keys(store, self.required_keys)

    def __len__(self) -> int:
        return len(self.store)

    @property
    def keys(self) -> List[str]:
        return self.store.keys

    @property
    def token_count(self) -> int:
        return self.store.token_count

    def __getitem__(self, index: int):
        raise NotImplementedError


class DatasetFactory(BaseFactory["BaseDataset"]):
    STREAM_TYPES = ("seq", "sft")

    @classmethod
    def load(cls, train_type: str, load_path: Optional[str] = None, window_size: int = 0, stride: Optional[int] = None,
             storage_type: Optional[str] = None, tokenizer_path: Optional[str] = None, max_len: int = 2048,
             store: Optional[Store] = None, **kwargs) -> "BaseDataset":
        """Build (or accept) a store and bind the dataset registered under ``train_type`` to it."""
        if store is not None:
            return cls.create(train_type, store=store)
        if load_path is None:
            raise ValueError("Either load_path or store must be provided")
        storage_type = storage_type or detect_format(load_path)
        window = window_size if train_type in cls.STREAM_TYPES else 0
        store = StoreFactory.create(storage_type, window_size=window, stride=(stride or window_size) or window)
        processor = cls._lazy_processor(train_type, storage_type, tokenizer_path, max_len)
        if processor is not None:
            store.load(load_path, processor=processor, **kwargs)
        elif storage_type == "jsonl":
            transform = cls._jsonl_transform(load_path, tokenizer_path)
            if transform is None and cls._is_pretokenized(train_type, load_path):
                # shards written by the preprocessing pipeline with storage_format "jsonl": token ids, not text
                store.load(load_path, processor=pretokenized_processor, **kwargs)
                return cls.create(train_type, store=store)
            if transform is None:
                raise FileNotFoundError(
                    "JSONL dataset config not found. Expected dataset_config.json alongside *.jsonl files, pass "
                    "tokenizer_path= for the built-in messages config, or use processor= for lazy tokenisation.")
            store.load(load_path, transform=transform, **kwargs)
        else:
            store.load(load_path, **kwargs)
        return cls.create(train_type, store=store)

    @classmethod
    def _is_pretokenized(cls, train_type: str, path: str) -> bool:
        """True when the first record already holds id lists under every key the dataset type needs."""
        from astrai_b200.data.storage import JsonlSource

        try:
            required = cls._entries[train_type].required_keys
        except (KeyError, AttributeError):
            return False
        records = JsonlSource(path).load()
        if not records or not required:
            return False
        first = records[0]
        return all(isinstance(first.get(k), list) for k in required)

    @staticmethod
    def _lazy_processor(train_type, storage_type, tokenizer_path, max_len) -> Optional[Callable]:
        if tokenizer_path is None or storage_type != "jsonl" or train_type != "dpo":
            return None
        from astrai_b200.tokenize import AutoTokenizer

        return partial(dpo_processor, tokenizer=AutoTokenizer.from_pretrained(tokenizer_path), max_len=max_len)

    @staticmethod
    def _jsonl_transform(path: str, tokenizer_path: Optional[str]):
        from astrai_b200.config import PipelineConfig
        from astrai_b200.preprocessing.transform import TokenizeTransform

        root = Path(path)
        cfg = root / "dataset_config.json" if root.is_dir() else None
        if cfg is not None and cfg.exists():
            return TokenizeTransform.from_config_file(str(cfg))
        if tokenizer_path:
            return TokenizeTransform(PipelineConfig.from_dict(DEFAULT_MESSAGES_CONFIG), tokenizer_path)
        return None


@DatasetFactory.register("seq")
class SEQDataset(BaseDataset):
    required_keys = ["sequence"]

    def __getitem__(self, index: int):
        b, e = self.store.sample_window(index)
        return {"input_ids": self.store.fetch(b, e, "sequence").long(),
                "target_ids": self.store.fetch(b + 1, e + 1, "sequence").long()}


@DatasetFactory.register("sft")
class SFTDataset(BaseDataset):
    required_keys = ["sequence", "loss_mask", "position_ids"]

    def __getitem__(self, index: int):
        b, e = self.store.sample_window(index)
        f = self.store.fetch
        return {"input_ids": f(b, e, "sequence").long(), "target_ids": f(b + 1, e + 1, "sequence").long(),
                "position_ids": f(b, e, "position_ids").long(), "loss_mask": f(b + 1, e + 1, "loss_mask").bool()}


@DatasetFactory.register("dpo")
class DPODataset(BaseDataset):
    required_keys = ["chosen", "rejected", "chosen_mask", "rejected_mask"]

    def __getitem__(self, index: int):
        rec = self.store.fetch_record(index, self.required_keys)
        return {"chosen": rec["chosen"].long(), "rejected": rec["rejected"].long(),
                "chosen_mask": rec["chosen_mask"].bool(), "rejected_mask": rec["rejected_mask"].bool()}


@DatasetFactory.register("grpo")
class GRPODataset(BaseDataset):
    required_keys = ["prompts", "responses", "masks", "rewards"]

    def __getitem__(self, index: int):
        rec = self.store.fetch_record(index, self.required_keys)
        return {"prompts": rec["prompts"].long(), "responses": [r.long() for r in rec["responses"]],
                "masks": [m.bool() for m in rec["masks"]], "rewards": rec["rewards"].float()}


class SyntheticTokenDataset(Dataset):
    """``num_samples`` packed sequences of uniform random token ids (deterministic per index), seq strategy layout."""

    def __init__(self, num_samples: int, seq_len: int, vocab_size: int, seed: int = 0):
        self.num_samples, self.seq_len, self.vocab_size, self.seed = num_samples, seq_len, vocab_size, seed

    def __len__(self):
        return self.num_samples

    def __getitem__(self, index: int):
        g = torch.Generator().manual_seed(self.seed * 1_000_003 + index)
        ids = torch.randint(0, self.vocab_size, (self.seq_len + 1,), generator=g)
        return {"input_ids": ids[:-1], "target_ids": ids[1:]}
