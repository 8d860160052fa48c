"""MMLU by answer-letter log-likelihood (reference: ``scripts/eval/evaluate_mmlu.py``).

Data layout: ``<data_dir>/<split>/<subject>_<split>.csv`` with rows ``question, A, B, C, D, answer`` (no header).
Each question is rendered through the chat template, the prompt ends right before the answer letter, and the score of a
choice is the log-probability of its letter token as the next token.  ``--permute`` shuffles the choices per item
(seeded) to cancel position bias.
"""

from __future__ import annotations

import argparse
import csv
import glob
import os
import random
from typing import Dict, List, Tuple

import torch

from astrai_b200.eval.common import batched, load_model_and_tokenizer, pad_right, save_json

LETTERS = ("A", "B", "C", "D")


def load_csv(path: str) -> List[dict]:
    rows = []
    with open(path, newline="", encoding="utf-8") as fh:
        for rec in csv.reader(fh):
            if len(rec) >= 6:
                rows.append({"question": rec[0], "choices": dict(zip(LETTERS, rec[1:5])), "answer": rec[5].strip()})
    return rows


def build_prompt(question: str, choices: Dict[str, str], subject: str) -> str:
    body = "\n".join(f"{k}. {v}" for k, v in choices.items())
    return (f"The following is a multiple choice question about {subject.replace('_', ' ')}.\n\n{question}\n{body}\n"
            "Answer with a single letter.")


def permute_choices(item: dict, rng: random.Random) -> Tuple[dict, str]:
    order = list(LETTERS)
    rng.shuffle(order)
    new = {LETTERS[i]: item["choices"][src] for i, src in enumerate(order)}
    return {**item, "choices": new}, LETTERS[order.index(item["answer"])]


@torch.no_grad()
def next_token_logprobs(model, rows: List[List[int]], device: str) -> torch.Tensor:
    """Log-softmax over the vocabulary at the position after each (right-padded) row: ``[B, V]``."""
    ids, mask = pad_right(rows)
    out = model(ids.to(device))
    logits = out["logits"] if "logits" in out else model.lm_head(out["hidden_states"])
    last = (mask.sum(1) - 1).to(device)
    return torch.log_softmax(logits[torch.arange(len(rows), device=device), last].float(), dim=-1)


def evaluate_subject(model, tokenizer, items: List[dict], subject: str, device: str, batch_size: int = 8, permute: bool = False,
                     seed: int = 0) -> Dict:
    rng = random.Random(seed)
    letter_ids = [tokenizer.encode(" " + l)[-1] for l in LETTERS]
    correct = 0
    for chunk in batched(items, batch_size):
        prompts, answers = [], []
        for it in chunk:
            it2, ans = permute_choices(it, rng) if permute else (it, it["answer"])
            text = tokenizer.apply_chat_template([{"role": "user", "content": build_prompt(it2["question"], it2["choices"], subject)}],
                                                 tokenize=False, add_generation_prompt=True)
            prompts.append(tokenizer.encode(text))
            answers.append(ans)
        lp = next_token_logprobs(model, prompts, device)[:, letter_ids]
        pred = lp.argmax(-1).tolist()
        correct += sum(LETTERS[p] == a for p, a in zip(pred, answers))
    return {"subject": subject, "n": len(items), "accuracy": correct / max(len(items), 1)}


def main(argv=None):
    ap = argparse.ArgumentParser(description="MMLU accuracy by answer-letter likelihood")
    ap.add_argument("--param_path", required=True)
    ap.add_argument("--data_dir", required=True)
    ap.add_argument("--split", default="test", choices=["test", "val"])
    ap.add_argument("--subjects", nargs="*", default=None)
    ap.add_argument("--batch_size", type=int, default=8)
    ap.add_argument("--max_items", type=int, default=None)
    ap.add_argument("--permute", action="store_true")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--device", default=None)
    ap.add_argument("--output", default=None)
    a = ap.parse_args(argv)
    model, tok, device = load_model_and_tokenizer(a.param_path, a.device)
    results = []
    for path in sorted(glob.glob(os.path.join(a.data_dir, a.split, f"*_{a.split}.csv"))):
        subject = os.path.basename(path)[: -len(f"_{a.split}.csv")]
        if a.subjects and subject not in a.subjects:
            continue
        results.append(evaluate_subject(model, tok, load_csv(path)[: a.max_items], subject, device, a.batch_size, a.permute, a.seed))
        print(results[-1])
    total = sum(r["n"] for r in results)
    summary = {"subjects": results, "n": total, "accuracy": sum(r["accuracy"] * r["n"] for r in results) / max(total, 1)}
    print({"n": total, "accuracy": summary["accuracy"]})
    save_json(a.output, summary)
    return summary


if __name__ == "__main__":
    main()
