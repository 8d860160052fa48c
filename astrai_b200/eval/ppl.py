"""Perplexity / token-loss statistics over JSON(L) text (reference: ``scripts/eval/evaluate_ppl.py``)."""

from __future__ import annotations

import argparse
import math
from typing import Dict, List

import torch

from astrai_b200.eval.common import batched, collect_files, load_items, load_model_and_tokenizer, pad_right, percentiles, save_json, token_nll


def score_texts(model, tokenizer, texts: List[str], device: str, max_len: int = 2048, batch_size: int = 8) -> Dict:
    losses: List[float] = []
    total, count = 0.0, 0
    rows = [tokenizer.encode(t)[:max_len] for t in texts]
    rows = [r for r in rows if len(r) >= 2]
    rows.sort(key=len)
    for chunk in batched(rows, batch_size):
        ids, mask = pad_right(list(chunk))
        nll = token_nll(model, ids.to(device)).float().cpu()
        valid = mask[:, 1:]
        per_doc = (nll * valid).sum(1) / valid.sum(1).clamp(min=1)
        losses += per_doc.tolist()
        total += float((nll * valid).sum())
        count += int(valid.sum())
    mean = total / max(count, 1)
    return {"documents": len(rows), "tokens": count, "mean_nll": mean, "ppl": math.exp(min(mean, 50.0)),
            "doc_loss": percentiles(losses)}


def main(argv=None):
    ap = argparse.ArgumentParser(description="Perplexity of a model on JSON(L) text files")
    ap.add_argument("--param_path", required=True)
    ap.add_argument("--input", required=True, help="file or directory of .jsonl / .json")
    ap.add_argument("--text_key", default="text")
    ap.add_argument("--max_len", type=int, default=2048)
    ap.add_argument("--batch_size", type=int, default=8)
    ap.add_argument("--max_items", type=int, default=None)
    ap.add_argument("--device", default=None)
    ap.add_argument("--output", default=None)
    a = ap.parse_args(argv)
    model, tok, device = load_model_and_tokenizer(a.param_path, a.device)
    report = {}
    for path in collect_files(a.input):
        texts = [str(it[a.text_key]) for it in load_items(path) if a.text_key in it][: a.max_items]
        report[path] = score_texts(model, tok, texts, device, a.max_len, a.batch_size)
        print(path, report[path])
    save_json(a.output, report)
    return report


if __name__ == "__main__":
    main()
