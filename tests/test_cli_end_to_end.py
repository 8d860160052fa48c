"""The command-line tools chained as a user would: preprocess JSONL chats, train on the shards, resume, generate."""

import json
import os

import pytest
import torch
from click.testing import CliRunner

from helpers import TINY, build_tokenizer_dir


@pytest.fixture(scope="module")
def workspace(tmp_path_factory):
    root = tmp_path_factory.mktemp("cli")
    params = build_tokenizer_dir(str(root / "params"))
    with open(os.path.join(params, "config.json"), "w") as fh:
        json.dump({**TINY, "vocab_size": 512}, fh)
    chats = root / "chats.jsonl"
    with open(chats, "w") as fh:
        for i in range(48):
            fh.write(json.dumps({"messages": [{"role": "user", "content": f"question number {i}"},
                                              {"role": "assistant", "content": "the answer is " + "yes " * (i % 4 + 1)}]}) + "\n")
    pipeline = root / "pipeline.json"
    pipeline.write_text(json.dumps({
        "input": {"sections": [{"field": "messages", "action": "$role", "template": True}]},
        "mask": {"user": "mask", "assistant": "train"},
        "preprocessing": {"packing_strategy": "bfd", "max_packed_len": 64, "batch_size": 16},
        "output": {"position_ids_mode": "doc_reset"}}))
    return {"root": root, "params": params, "chats": chats, "pipeline": pipeline}


def _train_args(ws, ckpt, *extra, param_path=None):
    return ["--train_type", "sft", "--data_root_path", str(ws["root"] / "shards"), "--param_path", str(param_path or ws["params"]),
            "--device_type", "cpu", "--backend", "gloo", "--parallel_mode", "none", "--nprocs", "1", "--optimizer", "fused_adamw",
            "--num_workers", "0", "--no-pin_memory", "--window_size", "32", "--batch_per_device", "2", "--ckpt_dir", str(ckpt),
            "--ckpt_interval", "4", "--metrics", "loss", "--metrics", "lr", *extra]


def test_preprocess_command_writes_shards(workspace):
    from astrai_b200.cli.preprocess import preprocess_command

    ws = workspace
    res = CliRunner().invoke(preprocess_command, [str(ws["chats"]), "-o", str(ws["root"] / "shards"), "-c", str(ws["pipeline"]),
                                                  "--tokenizer_path", ws["params"], "--batch_size", "5"])
    assert res.exit_code == 0, res.output
    assert "48 record(s) kept" in res.output
    shard = ws["root"] / "shards" / "__default__" / "shard_0000"
    assert sorted(p.name for p in shard.iterdir() if p.suffix == ".bin") == ["loss_mask.bin", "position_ids.bin", "sequence.bin"]


def test_preprocess_command_checks_its_arguments(workspace):
    from astrai_b200.cli.preprocess import preprocess_command

    ws = workspace
    res = CliRunner().invoke(preprocess_command, [str(ws["chats"]), "-o", str(ws["root"] / "x"), "-c", str(ws["pipeline"]), "--batch_size", "0"])
    assert res.exit_code == 2 and "batch_size" in res.output
    res = CliRunner().invoke(preprocess_command, ["-o", str(ws["root"] / "x"), "-c", str(ws["pipeline"])])
    assert res.exit_code == 2  # no input files
    res = CliRunner().invoke(preprocess_command, [str(ws["root"] / "missing.jsonl"), "-o", str(ws["root"] / "x"), "-c", str(ws["pipeline"])])
    assert res.exit_code == 2


def test_train_command_trains_checkpoints_and_resumes(workspace):
    from astrai_b200.cli.train import train_command
    from astrai_b200.serialization import Checkpoint, latest_complete

    ws = workspace
    if not (ws["root"] / "shards").exists():
        test_preprocess_command_writes_shards(ws)
    ckpt = ws["root"] / "ckpt"
    res = CliRunner().invoke(train_command, _train_args(ws, ckpt))
    assert res.exit_code == 0, (res.output, res.exception)
    assert "training plan:" in res.output
    first = Checkpoint.load(latest_complete(ckpt))
    assert first.consumed_samples > 0 and {"optimizer", "scheduler"} <= set(first.extra)
    assert first.config["vocab_size"] == 512
    rows = [json.loads(line) for line in open(latest_complete(ckpt) / "metric.jsonl")]  # every file holds the log so far
    steps = [r for r in rows if r["type"] == "step"]
    assert steps and all({"loss", "lr"} <= set(r) and "grad_norm" not in r for r in steps)
    assert sorted(r["step"] for r in steps) == list(range(1, first.consumed_samples // 2 + 1))

    # a second epoch on top of the first one, resumed from the checkpoint the first run ended with
    res = CliRunner().invoke(train_command, _train_args(ws, ckpt, "--n_epoch", "2", "--resume", param_path=latest_complete(ckpt)))
    assert res.exit_code == 0, (res.output, res.exception)
    second = Checkpoint.load(latest_complete(ckpt))
    assert second.consumed_samples == 2 * first.consumed_samples
    assert any(not torch.equal(second.state_dict[k], first.state_dict[k]) for k in first.state_dict)


def test_generate_command_answers_every_question(workspace):
    from astrai_b200.cli.generate import generate_command
    from astrai_b200.config import AutoRegressiveLMConfig
    from astrai_b200.models import AutoRegressiveLM

    ws = workspace
    model_dir = ws["root"] / "model"
    build_tokenizer_dir(str(model_dir))
    torch.manual_seed(0)
    AutoRegressiveLM(AutoRegressiveLMConfig(**{**TINY, "vocab_size": 512})).save_pretrained(str(model_dir))
    questions = ws["root"] / "q.jsonl"
    with open(questions, "w") as fh:
        for i in range(3):
            fh.write(json.dumps({"q": f"what is {i}?", "id": i}) + "\n")
        fh.write("\n")
    out = ws["root"] / "a.jsonl"
    res = CliRunner().invoke(generate_command, ["--param_path", str(model_dir), "--input_json_file", str(questions), "--output_json_file", str(out),
                                                "--question_key", "q", "--response_key", "a", "--device", "cpu", "--batch_size", "2",
                                                "--num_samples", "2", "--max_tokens", "4", "--max_seq_len", "64"])
    assert res.exit_code == 0, (res.output, res.exception)
    rows = [json.loads(line) for line in open(out)]
    assert [r["id"] for r in rows] == [0, 1, 2] and all(r["q"].startswith("what is") for r in rows)
    assert all(isinstance(r["a"], list) and len(r["a"]) == 2 and all(isinstance(t, str) for t in r["a"]) for r in rows)

    res = CliRunner().invoke(generate_command, ["--param_path", str(model_dir), "--input_json_file", str(questions), "--output_json_file", str(out),
                                                "--question_key", "q", "--device", "cpu", "--max_tokens", "3", "--max_seq_len", "64", "--temperature", "0"])
    assert res.exit_code == 0, (res.output, res.exception)
    rows = [json.loads(line) for line in open(out)]
    assert len(rows) == 3 and all(isinstance(r["response"], str) for r in rows)
