"""IFEval: verifiable instruction following (reference: ``scripts/eval/evaluate_ifeval.py``).

Each problem carries a prompt and a list of ``instruction_id_list`` / ``kwargs``; a response passes an instruction
when its checker returns True.  Reported: prompt-level accuracy (all instructions of a prompt pass) and
instruction-level accuracy.  The checkers are plain text predicates and are importable on their own.
"""

from __future__ import annotations

import argparse
import json
import re
from typing import Callable, Dict, List, Optional

from astrai_b200.eval.common import load_items, save_json

CHECKERS: Dict[str, Callable[[str, dict], bool]] = {}


def register(instruction_id: str):
    def deco(fn):
        CHECKERS[instruction_id] = fn
        return fn
    return deco


def _cmp(value: int, relation: Optional[str], target: int) -> bool:
    relation = (relation or "at least").lower()
    if relation in ("at least", ">="):
        return value >= target
    if relation in ("at most", "<=", "less than") :
        return value <= target if relation != "less than" else value < target
    return value == target


def count_words(text: str) -> int:
    return len(re.findall(r"\b\w+\b", text))


def count_sentences(text: str) -> int:
    return len([s for s in re.split(r"(?<=[.!?])\s+", text.strip()) if s])


def paragraphs(text: str) -> List[str]:
    return [p for p in re.split(r"\n\s*\n|\*\*\*", text.strip()) if p.strip()]


@register("keywords:existence")
def _(r, kw): return all(re.search(re.escape(k), r, re.I) for k in kw.get("keywords", []))
@register("keywords:frequency")
def _(r, kw): return _cmp(len(re.findall(re.escape(kw["keyword"]), r, re.I)), kw.get("relation"), int(kw["frequency"]))
@register("keywords:forbidden_words")
def _(r, kw): return not any(re.search(r"\b" + re.escape(k) + r"\b", r, re.I) for k in kw.get("forbidden_words", []))
@register("keywords:letter_frequency")
def _(r, kw): return _cmp(r.lower().count(str(kw["letter"]).lower()), kw.get("let_relation"), int(kw["let_frequency"]))
@register("detectable_content:number_placeholders")
def _(r, kw): return len(re.findall(r"\[[^\[\]]+\]", r)) >= int(kw["num_placeholders"])
@register("detectable_content:postscript")
def _(r, kw): return re.search(r"^\s*" + re.escape(kw.get("postscript_marker", "P.S.")), r, re.I | re.M) is not None
@register("detectable_format:number_bullet_lists")
def _(r, kw): return len(re.findall(r"^\s*[\*\-]\s+\S", r, re.M)) == int(kw["num_bullets"])
@register("detectable_format:number_highlighted_sections")
def _(r, kw): return len(re.findall(r"\*[^\n\*]+\*", r)) >= int(kw["num_highlights"])
@register("detectable_format:multiple_sections")
def _(r, kw): return len(re.findall(r"^\s*" + re.escape(kw.get("section_spliter", "Section")) + r"\s*\d+", r, re.M | re.I)) >= int(kw["num_sections"])
@register("detectable_format:title")
def _(r, kw): return re.search(r"<<[^\n]+>>", r) is not None
@register("detectable_format:json_format")
def _(r, kw):
    text = re.sub(r"^```(?:json)?|```$", "", r.strip(), flags=re.M).strip()
    try:
        json.loads(text)
        return True
    except ValueError:
        return False
@register("detectable_format:general_punctuation")
def _(r, kw): return not any(mark and mark in r for mark in kw.get("punctuation_blacklist", []))
@register("detectable_format:number_highlighted_words")
def _(r, kw): return len(re.findall(r"\*[^\s\*](?:[^\*]*[^\s\*])?\*", r)) >= int(kw.get("num_highlights", 1))
@register("punctuation:no_comma")
def _(r, kw): return "," not in r
@register("startend:end_checker")
def _(r, kw): return r.strip().lower().endswith(str(kw["end_phrase"]).strip().lower())
@register("startend:start_checker")
def _(r, kw): return re.search(r"^\s*" + re.escape(str(kw["starter"])), r, re.M) is not None
@register("startend:quotation")
def _(r, kw): return len(r.strip()) > 1 and r.strip()[0] == '"' and r.strip()[-1] == '"'
@register("change_case:english_capital")
def _(r, kw): return r == r.upper() and any(c.isalpha() for c in r)
@register("change_case:english_lowercase")
def _(r, kw): return r == r.lower() and any(c.isalpha() for c in r)
@register("change_case:capital_word_frequency")
def _(r, kw): return _cmp(len([w for w in re.findall(r"\b[A-Za-z]+\b", r) if w.isupper()]), kw.get("capital_relation"), int(kw["capital_frequency"]))
@register("length_constraints:number_words")
def _(r, kw): return _cmp(count_words(r), kw.get("relation"), int(kw["num_words"]))
@register("length_constraints:number_sentences")
def _(r, kw): return _cmp(count_sentences(r), kw.get("relation"), int(kw["num_sentences"]))
@register("length_constraints:number_paragraphs")
def _(r, kw): return len(paragraphs(r)) == int(kw["num_paragraphs"])
@register("length_constraints:nth_paragraph_first_word")
def _(r, kw):
    ps = paragraphs(r)
    n = int(kw["nth_paragraph"])
    if len(ps) != int(kw["num_paragraphs"]) or not (1 <= n <= len(ps)):
        return False
    words = re.findall(r"\b\w+\b", ps[n - 1])
    return bool(words) and words[0].lower() == str(kw["first_word"]).lower()
@register("length_constraints:nth_word_checker")
def _(r, kw):
    words = re.findall(r"\b\w+\b", r)
    n = int(kw.get("nth_word", 1))
    return 1 <= n <= len(words) and words[n - 1].lower() == str(kw.get("target_word", "")).lower()
@register("combination:repeat_prompt")
def _(r, kw): return r.strip().lower().startswith(str(kw["prompt_to_repeat"]).strip().lower())
@register("combination:two_responses")
def _(r, kw):
    parts = [p.strip() for p in r.split("******")]
    return len(parts) == 2 and all(parts) and parts[0] != parts[1]


def verify_response(response: str, instruction_id: str, kwargs: dict) -> Optional[bool]:
    fn = CHECKERS.get(instruction_id)
    if fn is None:
        return None  # unknown instruction: not counted
    try:
        return bool(fn(response, {k: v for k, v in (kwargs or {}).items() if v is not None}))
    except (KeyError, ValueError, TypeError):
        return False


def score(problems: List[dict], responses: List[str]) -> Dict:
    prompt_ok = inst_ok = inst_n = 0
    for prob, resp in zip(problems, responses):
        verdicts = [verify_response(resp, iid, kw) for iid, kw in zip(prob["instruction_id_list"], prob.get("kwargs") or [{}] * len(prob["instruction_id_list"]))]
        verdicts = [v for v in verdicts if v is not None]
        inst_n += len(verdicts)
        inst_ok += sum(verdicts)
        prompt_ok += bool(verdicts) and all(verdicts)
    return {"prompts": len(problems), "prompt_accuracy": prompt_ok / max(len(problems), 1), "instructions": inst_n,
            "instruction_accuracy": inst_ok / max(inst_n, 1)}


def main(argv=None):
    ap = argparse.ArgumentParser(description="IFEval prompt- and instruction-level accuracy")
    ap.add_argument("--param_path", default="./params")
    ap.add_argument("--data_path", required=True)
    ap.add_argument("--output", default=None)
    ap.add_argument("--max_tokens", type=int, default=1024)
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--batch_size", type=int, default=16)
    ap.add_argument("--max_seq_len", type=int, default=4096)
    ap.add_argument("--max_items", type=int, default=None)
    a = ap.parse_args(argv)
    import torch

    from astrai_b200.inference import InferenceEngine
    from astrai_b200.models import AutoModel
    from astrai_b200.tokenize import AutoTokenizer

    problems = load_items(a.data_path)[: a.max_items]
    tok = AutoTokenizer.from_pretrained(a.param_path)
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    model = AutoModel.from_pretrained(a.param_path).to(dev, torch.bfloat16 if dev == "cuda" else torch.float32).eval()
    engine = InferenceEngine(model, tok, max_batch_size=a.batch_size, max_seq_len=a.max_seq_len)
    responses: List[str] = []
    try:
        for i in range(0, len(problems), a.batch_size):
            prompts = [tok.apply_chat_template([{"role": "user", "content": p["prompt"]}], tokenize=False, add_generation_prompt=True)
                       for p in problems[i:i + a.batch_size]]
            responses += engine.generate(prompts, max_tokens=a.max_tokens, temperature=a.temperature)
    finally:
        engine.shutdown()
    res = score(problems, responses)
    print(res)
    save_json(a.output, {"summary": res, "responses": responses})
    return res


if __name__ == "__main__":
    main()
