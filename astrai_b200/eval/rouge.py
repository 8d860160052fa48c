"""ROUGE-1 / ROUGE-2 / ROUGE-L between ``reference`` and ``candidate`` fields (reference: ``scripts/eval/evaluate_rouge.py``)."""

from __future__ import annotations

import argparse
import re
from collections import Counter
from typing import Dict, List

from astrai_b200.eval.common import load_items, save_json


def tokenize(text: str) -> List[str]:
    return re.findall(r"\w+", text.lower())


def _f1(p: float, r: float) -> float:
    return 0.0 if p + r == 0 else 2 * p * r / (p + r)


def rouge_n(ref: List[str], cand: List[str], n: int) -> Dict[str, float]:
    grams = lambda t: Counter(tuple(t[i:i + n]) for i in range(len(t) - n + 1))  # noqa: E731
    r, c = grams(ref), grams(cand)
    overlap = sum((r & c).values())
    p = overlap / max(sum(c.values()), 1)
    rec = overlap / max(sum(r.values()), 1)
    return {"precision": p, "recall": rec, "f1": _f1(p, rec)}


def lcs(x: List[str], y: List[str]) -> int:
    prev = [0] * (len(y) + 1)
    for xi in x:
        cur = [0]
        for j, yj in enumerate(y):
            cur.append(prev[j] + 1 if xi == yj else max(prev[j + 1], cur[j]))
        prev = cur
    return prev[-1]


def rouge_l(ref: List[str], cand: List[str]) -> Dict[str, float]:
    n = lcs(ref, cand)
    p, r = n / max(len(cand), 1), n / max(len(ref), 1)
    return {"precision": p, "recall": r, "f1": _f1(p, r)}


def compute_rouge(reference: str, candidate: str) -> Dict[str, Dict[str, float]]:
    ref, cand = tokenize(reference), tokenize(candidate)
    return {"rouge1": rouge_n(ref, cand, 1), "rouge2": rouge_n(ref, cand, 2), "rougeL": rouge_l(ref, cand)}


def evaluate_file(path: str, ref_key: str = "reference", cand_key: str = "candidate") -> Dict:
    scores = [compute_rouge(str(it[ref_key]), str(it[cand_key])) for it in load_items(path) if ref_key in it and cand_key in it]
    out = {"items": len(scores)}
    for name in ("rouge1", "rouge2", "rougeL"):
        out[name] = {k: sum(s[name][k] for s in scores) / max(len(scores), 1) for k in ("precision", "recall", "f1")}
    return out


def main(argv=None):
    ap = argparse.ArgumentParser(description="ROUGE scores of a JSONL file")
    ap.add_argument("--data_path", required=True)
    ap.add_argument("--ref_key", default="reference")
    ap.add_argument("--cand_key", default="candidate")
    ap.add_argument("--output", default=None)
    a = ap.parse_args(argv)
    res = evaluate_file(a.data_path, a.ref_key, a.cand_key)
    print(res)
    save_json(a.output, res)
    return res


if __name__ == "__main__":
    main()
