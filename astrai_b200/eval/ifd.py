"""Instruction-following difficulty (IFD) of SFT pairs (reference: ``scripts/eval/evaluate_ifd.py``).

``IFD = loss(response | instruction) / loss(response)``: values near 1 mean the instruction does not help the model
predict the response (hard or noisy sample), small values mean an easy sample.
"""

from __future__ import annotations

import argparse
from typing import Dict, List

import torch

from astrai_b200.eval.common import collect_files, load_items, load_model_and_tokenizer, save_json, token_nll


def trim(context: List[int], response: List[int], max_len: int):
    """Keep the response (up to max_len - 1 tokens) and as much of the context's tail as still fits."""
    response = response[: max_len - 1]
    room = max_len - len(response)
    return context[-room:] if room > 0 else context[-1:], response


@torch.no_grad()
def ifd_score(model, tokenizer, instruction: str, response: str, device: str, max_len: int = 2048) -> Dict[str, float]:
    ctx = tokenizer.apply_chat_template([{"role": "user", "content": instruction}], tokenize=True, add_generation_prompt=True)
    resp = tokenizer.encode(response)
    if not resp:
        return {"ifd": float("nan"), "cond_loss": float("nan"), "resp_loss": float("nan")}
    ctx, resp = trim(list(ctx), list(resp), max_len)
    both = torch.tensor([ctx + resp], dtype=torch.long, device=device)
    cond = token_nll(model, both)[0, len(ctx) - 1:].mean().item()
    bos = getattr(tokenizer, "bos_token_id", None)
    alone_ids = ([bos] if bos is not None else [resp[0]]) + resp
    alone = token_nll(model, torch.tensor([alone_ids], dtype=torch.long, device=device))[0].mean().item()
    return {"ifd": cond / max(alone, 1e-8), "cond_loss": cond, "resp_loss": alone}


def main(argv=None):
    ap = argparse.ArgumentParser(description="IFD scores for instruction / response pairs")
    ap.add_argument("--param_path", required=True)
    ap.add_argument("--input", required=True)
    ap.add_argument("--instruction_key", default="instruction")
    ap.add_argument("--response_key", default="output")
    ap.add_argument("--max_len", type=int, default=2048)
    ap.add_argument("--max_items", type=int, default=None)
    ap.add_argument("--device", default=None)
    ap.add_argument("--output", default=None)
    a = ap.parse_args(argv)
    model, tok, device = load_model_and_tokenizer(a.param_path, a.device)
    rows = []
    for path in collect_files(a.input):
        for it in load_items(path)[: a.max_items]:
            if a.instruction_key in it and a.response_key in it:
                rows.append({**it, **ifd_score(model, tok, str(it[a.instruction_key]), str(it[a.response_key]), device, a.max_len)})
    ok = [r["ifd"] for r in rows if r["ifd"] == r["ifd"]]
    summary = {"items": len(rows), "mean_ifd": sum(ok) / max(len(ok), 1)}
    print(summary)
    save_json(a.output, {"summary": summary, "rows": rows})
    return summary


if __name__ == "__main__":
    main()
