"""HumanEval pass@k (reference: ``scripts/eval/evaluate_humaneval.py``).

Samples ``num_samples`` completions per problem through the inference engine, executes ``prompt + completion + test``
in a child Python process with a time limit, and reports the unbiased ``pass@k = 1 - C(n-c, k) / C(n, k)``.
"""

from __future__ import annotations

import argparse
import math
import os
import subprocess
import sys
import tempfile
from typing import Dict, List, Optional

from astrai_b200.eval.common import load_items, save_json

STOP_MARKERS = ("\ndef ", "\nclass ", "\nif __name__", "\nprint(", "\n#", "```")


def trim_stop(text: str) -> str:
    cut = len(text)
    for marker in STOP_MARKERS:
        i = text.find(marker)
        if i >= 0:
            cut = min(cut, i)
    return text[:cut]


def extract_body(code: str, entry_point: str) -> Optional[str]:
    """If the model repeated the signature, keep only what follows it."""
    marker = f"def {entry_point}"
    i = code.find(marker)
    if i < 0:
        return code
    j = code.find("\n", code.find(":", i))
    return code[j + 1:] if j >= 0 else None


def pass_at_k(n: int, c: int, k: int) -> float:
    if n - c < k:
        return 1.0
    return 1.0 - math.prod((n - c - i) / (n - i) for i in range(k))


def execute_one(program: str, timeout: float) -> bool:
    with tempfile.NamedTemporaryFile("w", suffix=".py", delete=False) as fh:
        fh.write(program)
        path = fh.name
    try:
        proc = subprocess.run([sys.executable, "-I", path], capture_output=True, timeout=timeout)
        return proc.returncode == 0
    except subprocess.TimeoutExpired:
        return False
    finally:
        os.unlink(path)


def score_problem(item: dict, completions: List[str], timeout: float) -> int:
    passed = 0
    for comp in dict.fromkeys(completions):  # identical completions are executed once
        body = extract_body(trim_stop(comp), item["entry_point"]) or ""
        program = item["prompt"] + body + "\n\n" + item["test"] + f"\n\ncheck({item['entry_point']})\n"
        if execute_one(program, timeout):
            passed += completions.count(comp)
    return passed


def main(argv=None):
    ap = argparse.ArgumentParser(description="HumanEval pass@k")
    ap.add_argument("--param_path", default="./params")
    ap.add_argument("--data_path", default="./humaneval/HumanEval.jsonl")
    ap.add_argument("--output", default=None)
    ap.add_argument("--k", type=int, nargs="+", default=[1, 10, 100])
    ap.add_argument("--num_samples", type=int, default=200)
    ap.add_argument("--max_tokens", type=int, default=512)
    ap.add_argument("--temperature", type=float, default=0.8)
    ap.add_argument("--top_p", type=float, default=0.95)
    ap.add_argument("--top_k", type=int, default=50)
    ap.add_argument("--batch_size", type=int, default=64)
    ap.add_argument("--max_seq_len", type=int, default=4096)
    ap.add_argument("--test_timeout", type=float, default=3.0)
    ap.add_argument("--problems", type=int, nargs="+", default=None)
    a = ap.parse_args(argv)
    import torch

    from astrai_b200.inference import InferenceEngine
    from astrai_b200.models import AutoModel
    from astrai_b200.tokenize import AutoTokenizer

    items = load_items(a.data_path)
    if a.problems:
        items = [items[i] for i in a.problems]
    tok = AutoTokenizer.from_pretrained(a.param_path)
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    model = AutoModel.from_pretrained(a.param_path).to(dev, torch.bfloat16 if dev == "cuda" else torch.float32).eval()
    engine = InferenceEngine(model, tok, max_batch_size=a.batch_size, max_seq_len=a.max_seq_len)
    results: Dict[str, Dict] = {}
    try:
        for it in items:
            comps: List[str] = []
            while len(comps) < a.num_samples:
                n = min(a.batch_size, a.num_samples - len(comps))
                comps += engine.generate([it["prompt"]] * n, max_tokens=a.max_tokens, temperature=a.temperature, top_p=a.top_p, top_k=a.top_k)
            c = score_problem(it, comps, a.test_timeout)
            results[it["task_id"]] = {"n": len(comps), "c": c}
            print(it["task_id"], results[it["task_id"]])
    finally:
        engine.shutdown()
    summary = {f"pass@{k}": sum(pass_at_k(r["n"], r["c"], k) for r in results.values()) / max(len(results), 1)
               for k in a.k if k <= a.num_samples}
    print(summary)
    save_json(a.output, {"summary": summary, "problems": results})
    return summary


if __name__ == "__main__":
    main()
