"""The evaluation command lines and the demo programs, run as a user runs them, on a tiny random model on the CPU."""

import builtins
import csv
import json
import logging
import math
import sys

import pytest
import torch

from helpers import TINY, build_tokenizer_dir


@pytest.fixture(scope="module")
def model_dir(tmp_path_factory):
    from astrai_b200.config import AutoRegressiveLMConfig
    from astrai_b200.models import AutoRegressiveLM

    path = tmp_path_factory.mktemp("tools") / "model"
    build_tokenizer_dir(str(path))
    torch.manual_seed(0)
    AutoRegressiveLM(AutoRegressiveLMConfig(**{**TINY, "vocab_size": 512, "max_position_embeddings": 256})).save_pretrained(str(path))
    return str(path)


def _jsonl(path, rows):
    with open(path, "w") as fh:
        for r in rows:
            fh.write(json.dumps(r) + "\n")
    return str(path)


def test_ppl_command(model_dir, tmp_path):
    from astrai_b200.eval import ppl

    data = tmp_path / "texts"
    data.mkdir()
    _jsonl(data / "a.jsonl", [{"text": "the quick brown fox " * 3}, {"text": "hello world"}, {"other": "ignored"}, {"text": "x"}])
    (data / "b.json").write_text(json.dumps([{"text": "user assistant system " * 2}]))
    out = tmp_path / "ppl.json"
    report = ppl.main(["--param_path", model_dir, "--input", str(data), "--device", "cpu", "--batch_size", "2", "--max_len", "24", "--output", str(out)])
    assert len(report) == 2 and json.loads(out.read_text()).keys() == report.keys()
    a = report[str(data / "a.jsonl")]
    assert a["documents"] == 2  # the one-token text has nothing to predict
    assert a["ppl"] == pytest.approx(math.exp(a["mean_nll"])) and 100 < a["ppl"] < 2000  # near-uniform over 512 tokens
    assert set(a["doc_loss"]) == {"p50", "p90", "p95", "p99"}


def test_ppl_does_not_depend_on_the_batching(model_dir):
    from astrai_b200.eval.common import load_model_and_tokenizer
    from astrai_b200.eval.ppl import score_texts

    model, tok, device = load_model_and_tokenizer(model_dir, "cpu")
    texts = ["the quick brown fox", "hello world hello", "system", "a much longer line of text to score " * 2]
    one = score_texts(model, tok, texts, device, batch_size=1)
    many = score_texts(model, tok, texts, device, batch_size=4)
    assert one["tokens"] == many["tokens"] and one["mean_nll"] == pytest.approx(many["mean_nll"], rel=1e-5)


def test_ifd_command(model_dir, tmp_path):
    from astrai_b200.eval import ifd

    src = _jsonl(tmp_path / "pairs.jsonl", [{"instruction": "say hello", "output": "hello world"}, {"instruction": "nothing", "output": ""},
                                            {"instruction": "no output key"}])
    out = tmp_path / "ifd.json"
    summary = ifd.main(["--param_path", model_dir, "--input", src, "--device", "cpu", "--output", str(out)])
    saved = json.loads(out.read_text().replace("NaN", "null"))
    assert summary["items"] == 2 and len(saved["rows"]) == 2
    first = saved["rows"][0]
    assert first["ifd"] == pytest.approx(first["cond_loss"] / first["resp_loss"]) and 0.5 < first["ifd"] < 2.0
    assert saved["rows"][1]["ifd"] is None  # an empty response has no loss


def test_ifd_trim_keeps_the_response_and_the_end_of_the_context():
    from astrai_b200.eval.ifd import trim

    ctx, resp = trim(list(range(10)), list(range(100, 104)), max_len=8)
    assert resp == [100, 101, 102, 103] and ctx == [6, 7, 8, 9]
    ctx, resp = trim(list(range(10)), list(range(100, 120)), max_len=8)
    assert len(resp) == 7 and ctx == [9]


def test_mmlu_command(model_dir, tmp_path):
    from astrai_b200.eval import mmlu

    split = tmp_path / "mmlu" / "test"
    split.mkdir(parents=True)
    for subject, n in (("algebra", 5), ("history", 3)):
        with open(split / f"{subject}_test.csv", "w", newline="") as fh:
            w = csv.writer(fh)
            for i in range(n):
                w.writerow([f"question {i} of {subject}?", "one", "two", "three", "four", "ABCD"[i % 4]])
    out = tmp_path / "mmlu.json"
    res = mmlu.main(["--param_path", model_dir, "--data_dir", str(tmp_path / "mmlu"), "--device", "cpu", "--batch_size", "2", "--output", str(out)])
    assert res["n"] == 8 and [s["subject"] for s in res["subjects"]] == ["algebra", "history"]
    assert res["accuracy"] == pytest.approx(sum(s["accuracy"] * s["n"] for s in res["subjects"]) / 8)
    only = mmlu.main(["--param_path", model_dir, "--data_dir", str(tmp_path / "mmlu"), "--device", "cpu", "--subjects", "history", "--max_items", "2",
                      "--permute"])
    assert only["n"] == 2 and len(only["subjects"]) == 1


def test_rouge_command(tmp_path):
    from astrai_b200.eval import rouge

    src = _jsonl(tmp_path / "r.jsonl", [{"ref": "the cat sat on the mat", "hyp": "the cat sat on the mat"}, {"ref": "a b c d", "hyp": "x y z"}, {"ref": "skipped"}])
    out = tmp_path / "rouge.json"
    res = rouge.main(["--data_path", src, "--ref_key", "ref", "--cand_key", "hyp", "--output", str(out)])
    assert res["items"] == 2 and res["rouge1"]["f1"] == pytest.approx(0.5) and res["rougeL"]["recall"] == pytest.approx(0.5)
    assert json.loads(out.read_text()) == res


def test_analyze_weights_command(model_dir, tmp_path):
    from astrai_b200.eval import analyze_weights

    out = tmp_path / "w.json"
    res = analyze_weights.main(["--param_path", model_dir, "--filter", "q_proj", "--output", str(out)])
    assert len(res) == TINY["num_hidden_layers"] and all("q_proj" in k for k in res)
    m = next(iter(res.values()))
    assert 1.0 <= m["stable_rank"] <= m["effective_rank"] + 1e-3 <= m["max_rank"] + 2e-3 and 0 < m["rank90_fraction"] <= 1


def test_ifeval_command(model_dir, tmp_path):
    from astrai_b200.eval import ifeval

    src = _jsonl(tmp_path / "if.jsonl", [
        {"prompt": "answer in lower case", "instruction_id_list": ["change_case:english_lowercase"], "kwargs": [{}]},
        {"prompt": "write at least 500 words", "instruction_id_list": ["length_constraints:number_words", "not:a_known_rule"],
         "kwargs": [{"relation": "at least", "num_words": 500}, {}]},
        {"prompt": "dropped by max_items", "instruction_id_list": [], "kwargs": []}])
    out = tmp_path / "if.json"
    res = ifeval.main(["--param_path", model_dir, "--data_path", src, "--max_tokens", "5", "--batch_size", "2", "--max_seq_len", "128", "--max_items", "2",
                       "--output", str(out)])
    saved = json.loads(out.read_text())
    assert res["prompts"] == 2 and res["instructions"] == 2 and len(saved["responses"]) == 2  # the unknown rule is not counted
    assert 0.0 <= res["instruction_accuracy"] <= 0.5  # five tokens are never 500 words


def test_humaneval_command(model_dir, tmp_path):
    from astrai_b200.eval import humaneval

    problem = {"task_id": "T/0", "entry_point": "add", "prompt": "def add(a, b):\n", "test": "def check(f):\n    assert f(1, 2) == 3\n"}
    src = _jsonl(tmp_path / "he.jsonl", [problem, {**problem, "task_id": "T/1"}])
    out = tmp_path / "he.json"
    res = humaneval.main(["--param_path", model_dir, "--data_path", src, "--num_samples", "3", "--k", "1", "2", "10", "--max_tokens", "4", "--batch_size", "2",
                          "--max_seq_len", "64", "--test_timeout", "10", "--problems", "1", "--output", str(out)])
    saved = json.loads(out.read_text())
    assert set(res) == {"pass@1", "pass@2"}  # k beyond the sample count is left out
    assert list(saved["problems"]) == ["T/1"] and saved["problems"]["T/1"]["n"] == 3
    assert res["pass@1"] == pytest.approx(saved["problems"]["T/1"]["c"] / 3)


def test_humaneval_scoring_runs_the_tests_once_per_distinct_completion(monkeypatch):
    from astrai_b200.eval import humaneval

    item = {"entry_point": "add", "prompt": "def add(a, b):\n", "test": "def check(f):\n    assert f(1, 2) == 3\n"}
    runs = []
    real = humaneval.execute_one
    monkeypatch.setattr(humaneval, "execute_one", lambda program, timeout: runs.append(program) or real(program, timeout))
    good, bad = "    return a + b\n", "    return a - b\n"
    assert humaneval.score_problem(item, [good, bad, good, good], timeout=20) == 3
    assert len(runs) == 2


# ---- demo programs -------------------------------------------------------------------------------------------------------

def _run_demo(module, monkeypatch, model_dir, *extra):
    monkeypatch.setattr(sys, "argv", [module.__name__, "--param_path", model_dir, "--device", "cpu", "--max_seq_len", "128", "--max_batch_size", "4",
                                      "--max_tokens", "4", *extra])
    module.main()


def test_single_prompt_demo(model_dir, monkeypatch, capsys):
    from astrai_b200.demo import generate_ar

    _run_demo(generate_ar, monkeypatch, model_dir, "--prompt", "hello", "--temperature", "0")
    first = capsys.readouterr().out
    _run_demo(generate_ar, monkeypatch, model_dir, "--prompt", "hello", "--temperature", "0")
    assert first and first == capsys.readouterr().out  # greedy decoding repeats itself


def test_batch_demo_prints_one_answer_per_prompt(model_dir, monkeypatch, capsys):
    from astrai_b200.demo import generate_batch

    _run_demo(generate_batch, monkeypatch, model_dir)
    out = capsys.readouterr().out
    assert [line[2:] for line in out.splitlines() if line.startswith("> ")] == generate_batch.PROMPTS


def test_chat_demo_streams_and_keeps_the_history(model_dir, monkeypatch, capsys):
    from astrai_b200.demo import _common, stream_chat

    typed = iter(["hello", "and again", ""])
    monkeypatch.setattr(builtins, "input", lambda prompt="": next(typed))
    seen = []
    real = _common.chat_prompt
    monkeypatch.setattr(stream_chat, "chat_prompt", lambda tok, messages: seen.append([dict(m) for m in messages]) or real(tok, messages))
    _run_demo(stream_chat, monkeypatch, model_dir)
    assert capsys.readouterr().out.count("bot> ") == 2
    assert [len(m) for m in seen] == [1, 3] and [m["role"] for m in seen[1]] == ["user", "assistant", "user"]


def test_chat_demo_ends_at_end_of_input(model_dir, monkeypatch, capsys):
    from astrai_b200.demo import stream_chat

    def closed(prompt=""):
        raise EOFError

    monkeypatch.setattr(builtins, "input", closed)
    _run_demo(stream_chat, monkeypatch, model_dir)
    assert "bot>" not in capsys.readouterr().out


def test_download_demo_explains_a_missing_hub_client(monkeypatch):
    from astrai_b200.demo import download

    monkeypatch.setattr(sys, "argv", ["download", "--out", "nowhere"])
    monkeypatch.setitem(sys.modules, "huggingface_hub", None)  # importing it now fails
    with pytest.raises(SystemExit, match="huggingface_hub is not installed"):
        download.main()


# ---- small shared pieces -----------------------------------------------------------------------------------------------------

def test_logging_setup_is_idempotent_and_tags_the_rank(monkeypatch, capsys):
    from astrai_b200 import logging as alog

    logger = logging.getLogger(alog.LOGGER_NAME)
    old_handlers, old_level = list(logger.handlers), logger.level
    logger.handlers.clear()
    try:
        monkeypatch.setenv("ASTR_LOG_LEVEL", "warning")
        monkeypatch.setenv("RANK", "3")
        monkeypatch.setenv("WORLD_SIZE", "8")
        assert alog.setup_logging("DEBUG") is logger and logger.level == logging.WARNING  # the environment wins
        assert alog.setup_logging() is logger and len(logger.handlers) == 1
        logging.getLogger(alog.LOGGER_NAME + ".unit").warning("look at this")
        logging.getLogger(alog.LOGGER_NAME + ".unit").info("not shown")
        err = capsys.readouterr().err
        assert "rank= 3/8" in err and "look at this" in err and "not shown" not in err
    finally:
        logger.handlers[:] = old_handlers
        logger.setLevel(old_level)


def test_optimizer_and_scheduler_protocols():
    from astrai_b200.optim import FusedAdamW
    from astrai_b200.protocols import OptimizerProtocol, SchedulerProtocol
    from astrai_b200.trainer import SchedulerFactory

    opt = FusedAdamW(torch.nn.Linear(2, 2).parameters(), lr=1e-3)
    assert isinstance(opt, OptimizerProtocol) and isinstance(torch.optim.SGD(torch.nn.Linear(2, 2).parameters(), lr=1), OptimizerProtocol)
    assert isinstance(SchedulerFactory.create("cosine", opt, warmup_steps=1, lr_decay_steps=4), SchedulerProtocol)
    assert not isinstance(object(), OptimizerProtocol) and not isinstance(opt, SchedulerProtocol)


def test_eval_input_helpers(tmp_path):
    from astrai_b200.eval.common import collect_files, load_items, pad_right, percentiles

    (tmp_path / "deep").mkdir()
    _jsonl(tmp_path / "deep" / "b.jsonl", [{"a": 1}, {"a": 2}])
    (tmp_path / "a.json").write_text(json.dumps({"a": 3}))
    (tmp_path / "lines.json").write_text('{"a": 4}\n{"a": 5}\n')  # JSON lines under a .json name
    (tmp_path / "empty.jsonl").write_text("")
    files = collect_files(str(tmp_path))
    assert [f.split("/")[-1] for f in files] == ["b.jsonl", "empty.jsonl", "a.json", "lines.json"]
    assert collect_files(files[0]) == [files[0]]
    assert [load_items(f) for f in files] == [[{"a": 1}, {"a": 2}], [], [{"a": 3}], [{"a": 4}, {"a": 5}]]
    ids, mask = pad_right([[1, 2, 3], [4]], pad_id=9)
    assert ids.tolist() == [[1, 2, 3], [4, 9, 9]] and mask.tolist() == [[True, True, True], [True, False, False]]
    assert percentiles([]) == {} and percentiles([3.0, 1.0, 2.0], qs=(0, 50, 100)) == {"p0": 1.0, "p50": 2.0, "p100": 3.0}
