"""Evaluation helpers: ROUGE, IFEval checkers, pass@k, effective rank, perplexity / IFD / MMLU on a tiny model (CPU)."""

import math
import sys
from pathlib import Path

import pytest
import torch

sys.path.insert(0, str(Path(__file__).parent))


def test_rouge_scores():
    from astrai_b200.eval.rouge import compute_rouge, lcs

    s = compute_rouge("the cat sat on the mat", "the cat lay on the mat")
    assert s["rouge1"]["f1"] == pytest.approx(5 / 6) and s["rouge2"]["recall"] == pytest.approx(3 / 5)
    assert lcs("a b c d".split(), "a c d b".split()) == 3 and s["rougeL"]["f1"] == pytest.approx(5 / 6)
    assert compute_rouge("x", "")["rouge1"]["f1"] == 0.0


def test_ifeval_checkers_and_scoring():
    from astrai_b200.eval.ifeval import score, verify_response

    assert verify_response("Hello, world", "punctuation:no_comma", {}) is False
    assert verify_response("one two three", "length_constraints:number_words", {"relation": "at most", "num_words": 3}) is True
    assert verify_response('{"a": 1}', "detectable_format:json_format", {}) is True
    assert verify_response("* a\n* b", "detectable_format:number_bullet_lists", {"num_bullets": 2}) is True
    assert verify_response("<<Title>>\nbody", "detectable_format:title", {}) is True
    assert verify_response("x", "made:up", {}) is None
    res = score([{"instruction_id_list": ["punctuation:no_comma", "change_case:english_lowercase"], "kwargs": [{}, {}]},
                 {"instruction_id_list": ["startend:end_checker"], "kwargs": [{"end_phrase": "bye"}]}], ["all lower", "hello BYE"])
    assert res["prompt_accuracy"] == 1.0 and res["instructions"] == 3


def test_pass_at_k_and_code_helpers():
    from astrai_b200.eval.humaneval import execute_one, extract_body, pass_at_k, trim_stop

    assert pass_at_k(10, 0, 1) == 0.0 and pass_at_k(10, 10, 1) == 1.0
    assert pass_at_k(10, 3, 1) == pytest.approx(0.3) and pass_at_k(5, 1, 5) == 1.0
    assert trim_stop("    return 1\n\ndef other():\n    pass") == "    return 1\n"
    assert extract_body("def f(x):\n    return x\n", "f") == "    return x\n"
    assert execute_one("assert 1 + 1 == 2\n", 5.0) and not execute_one("raise SystemExit(3)\n", 5.0)


def test_effective_rank():
    from astrai_b200.eval.analyze_weights import effective_rank_metrics

    eye = effective_rank_metrics(torch.eye(8))
    assert eye["effective_rank"] == pytest.approx(8.0, rel=1e-4) and eye["stable_rank"] == pytest.approx(8.0, rel=1e-4)
    rank1 = effective_rank_metrics(torch.ones(6, 4))
    assert rank1["effective_rank"] == pytest.approx(1.0, abs=1e-3) and rank1["rank90_fraction"] == pytest.approx(0.25)


def test_model_scoring_on_tiny_model(tmp_path):
    from helpers import build_tokenizer_dir, tiny_config

    from astrai_b200.eval.common import token_nll
    from astrai_b200.eval.ifd import ifd_score, trim
    from astrai_b200.eval.mmlu import build_prompt, evaluate_subject, permute_choices
    from astrai_b200.eval.ppl import score_texts
    from astrai_b200.models import AutoRegressiveLM
    from astrai_b200.tokenize import AutoTokenizer

    tok = AutoTokenizer.from_pretrained(build_tokenizer_dir(str(tmp_path)))
    torch.manual_seed(0)
    model = AutoRegressiveLM(tiny_config(vocab_size=512, max_position_embeddings=256)).eval()
    ids = torch.randint(0, 512, (2, 12))
    nll = token_nll(model, ids)
    ref = -torch.log_softmax(model(ids[:, :-1])["logits"].float(), -1).gather(-1, ids[:, 1:, None]).squeeze(-1)
    assert torch.allclose(nll, ref, atol=1e-5)
    rep = score_texts(model, tok, ["hello world hello", "the quick brown fox", "x"], "cpu", batch_size=2)
    assert rep["documents"] >= 2 and rep["ppl"] == pytest.approx(math.exp(rep["mean_nll"]))
    out = ifd_score(model, tok, "say hello", "hello world", "cpu")
    assert out["ifd"] > 0 and out["cond_loss"] > 0
    assert trim(list(range(10)), list(range(5)), 8) == ([7, 8, 9], [0, 1, 2, 3, 4])
    item = {"question": "2+2?", "choices": {"A": "3", "B": "4", "C": "5", "D": "6"}, "answer": "B"}
    import random

    it2, ans = permute_choices(item, random.Random(1))
    assert it2["choices"][ans] == "4" and "2+2?" in build_prompt(item["question"], item["choices"], "elementary_math")
    res = evaluate_subject(model, tok, [item, item], "elementary_math", "cpu", batch_size=2)
    assert res["n"] == 2 and 0.0 <= res["accuracy"] <= 1.0


IFEVAL_CASES = [
    ("keywords:existence", {"keywords": ["alpha", "Beta"]}, "Alpha and beta are here", "only alpha"),
    ("keywords:frequency", {"keyword": "cat", "relation": "at least", "frequency": 2}, "cat, Cat!", "one cat"),
    ("keywords:forbidden_words", {"forbidden_words": ["bad"]}, "a badge is fine", "this is bad"),
    ("keywords:letter_frequency", {"letter": "z", "let_relation": "less than", "let_frequency": 2}, "zebra", "pizza"),
    ("detectable_content:number_placeholders", {"num_placeholders": 2}, "[name] lives at [address]", "[name] only"),
    ("detectable_content:postscript", {"postscript_marker": "P.S."}, "body\nP.S. one more thing", "body without it"),
    ("detectable_format:number_bullet_lists", {"num_bullets": 2}, "- a\n- b", "- a\n- b\n- c"),
    ("detectable_format:number_highlighted_sections", {"num_highlights": 2}, "*one* and *two*", "*one* only"),
    ("detectable_format:number_highlighted_words", {"num_highlights": 2}, "a *b* c *d e* f", "* not closed and *x*"),
    ("detectable_format:general_punctuation", {"punctuation_blacklist": ["!", ";"]}, "calm, quiet.", "loud!"),
    ("detectable_format:multiple_sections", {"section_spliter": "Part", "num_sections": 2}, "Part 1\nx\nPart 2\ny", "Part 1 only"),
    ("detectable_format:title", {}, "<<A title>>\ntext", "no title"),
    ("detectable_format:json_format", {}, '```json\n{"a": [1, 2]}\n```', "{not json}"),
    ("punctuation:no_comma", {}, "no commas here", "one, comma"),
    ("startend:end_checker", {"end_phrase": "The end."}, "story. the end.", "the end. not"),
    ("startend:start_checker", {"starter": "Dear team"}, "  Dear team, hello", "Hello, Dear team"),
    ("startend:quotation", {}, '"quoted"', 'not "quoted'),
    ("change_case:english_capital", {}, "ALL CAPS 123", "Not all caps"),
    ("change_case:english_lowercase", {}, "all lower 123", "Not lower"),
    ("change_case:capital_word_frequency", {"capital_relation": "at least", "capital_frequency": 2}, "NASA and ESA", "NASA only"),
    ("length_constraints:number_words", {"relation": "at least", "num_words": 3}, "one two three", "one two"),
    ("length_constraints:number_sentences", {"relation": "at most", "num_sentences": 2}, "One. Two.", "One. Two. Three."),
    ("length_constraints:number_paragraphs", {"num_paragraphs": 2}, "first\n\nsecond", "only one"),
    ("length_constraints:nth_paragraph_first_word", {"num_paragraphs": 2, "nth_paragraph": 2, "first_word": "then"}, "a b\n\nThen c", "a b\n\nc then"),
    ("length_constraints:nth_word_checker", {"nth_word": 3, "target_word": "fox"}, "the quick FOX jumps", "the quick brown fox"),
    ("combination:repeat_prompt", {"prompt_to_repeat": "Say hi"}, "say hi\nhi!", "hi! say hi"),
    ("combination:two_responses", {}, "one ****** two", "same ****** same"),
]


@pytest.mark.parametrize("instruction,kwargs,good,bad", IFEVAL_CASES, ids=[c[0] for c in IFEVAL_CASES])
def test_every_ifeval_instruction_accepts_and_rejects(instruction, kwargs, good, bad):
    from astrai_b200.eval.ifeval import verify_response

    assert verify_response(good, instruction, kwargs) is True
    assert verify_response(bad, instruction, kwargs) is False


def test_ifeval_covers_the_27_instruction_kinds():
    from astrai_b200.eval import ifeval

    registry = next(v for v in vars(ifeval).values() if isinstance(v, dict) and "punctuation:no_comma" in v)
    assert len(registry) == 27 and {c[0] for c in IFEVAL_CASES} == set(registry)
