"""Shared helpers of the eval scripts: model loading, JSON(L) input, batched causal scoring."""

from __future__ import annotations

import glob
import json
import os
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

import torch
from torch import Tensor


def load_model_and_tokenizer(param_path: str, device: Optional[str] = None, dtype: Optional[torch.dtype] = None):
    from astrai_b200.models import AutoModel
    from astrai_b200.tokenize import AutoTokenizer

    device = device or ("cuda" if torch.cuda.is_available() else "cpu")
    dtype = dtype or (torch.bfloat16 if device.startswith("cuda") else torch.float32)
    model = AutoModel.from_pretrained(param_path).to(device=device, dtype=dtype).eval()
    return model, AutoTokenizer.from_pretrained(param_path), device


def collect_files(path: str, patterns: Sequence[str] = ("*.jsonl", "*.json")) -> List[str]:
    if os.path.isfile(path):
        return [path]
    out: List[str] = []
    for pat in patterns:
        out += sorted(glob.glob(os.path.join(path, "**", pat), recursive=True))
    return out


def load_items(path: str) -> List[dict]:
    with open(path, encoding="utf-8") as fh:
        text = fh.read().strip()
    if not text:
        return []
    if path.endswith(".jsonl") or (text[0] != "[" and "\n" in text):
        return [json.loads(line) for line in text.splitlines() if line.strip()]
    data = json.loads(text)
    return data if isinstance(data, list) else [data]


def save_json(path: Optional[str], data) -> None:
    if path:
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
        with open(path, "w", encoding="utf-8") as fh:
            json.dump(data, fh, indent=2, ensure_ascii=False)


@torch.no_grad()
def token_nll(model, ids: Tensor) -> Tensor:
    """Per-position negative log-likelihood of ``ids[:, 1:]`` given the prefix: ``[B, S-1]`` fp32.

    Equal-length rows with no mask -> causal attention (a 2-D padding mask would make the forward non-causal, which is
    the reference's behaviour too; callers pad on the right and ignore the padded positions instead)."""
    from astrai_b200 import ops

    inner = getattr(model, "lm_head", None)
    if inner is not None and getattr(model, "supports_fused_head", False) and ids.is_cuda:
        hidden = model(ids[:, :-1], return_logits=False)["hidden_states"]
        return -ops.linear_token_logprobs(hidden, model.lm_head.weight, ids[:, 1:])
    logits = model(ids[:, :-1])["logits"].float()
    return -torch.log_softmax(logits, dim=-1).gather(-1, ids[:, 1:, None]).squeeze(-1)


def batched(items: Sequence, n: int) -> Iterable[Sequence]:
    for i in range(0, len(items), n):
        yield items[i:i + n]


def pad_right(rows: List[List[int]], pad_id: int = 0) -> Tuple[Tensor, Tensor]:
    width = max(len(r) for r in rows)
    ids = torch.full((len(rows), width), pad_id, dtype=torch.long)
    mask = torch.zeros((len(rows), width), dtype=torch.bool)
    for i, r in enumerate(rows):
        ids[i, : len(r)] = torch.tensor(r, dtype=torch.long)
        mask[i, : len(r)] = True
    return ids, mask


def percentiles(values: List[float], qs=(50, 90, 95, 99)) -> Dict[str, float]:
    if not values:
        return {}
    s = sorted(values)
    return {f"p{q}": s[min(len(s) - 1, int(round(q / 100 * (len(s) - 1))))] for q in qs}
