"""CLI surface: YAML precedence, dry-run plan, required options, runtime exports, step arithmetic."""

import json

from click.testing import CliRunner

from astrai_b200.cli import runtime
from astrai_b200.cli.train import compute_total_steps, scheduler_kwargs, train_command


def test_yaml_below_explicit_cli_above_defaults(tmp_path):
    cfg = tmp_path / "t.yaml"
    cfg.write_text("training:\n  max_lr: 1e-4\n  batch_per_device: 8\nparallel:\n  nprocs: 4\ndata:\n  data_root_path: /data\n"
                   "train_type: sft\nparam_path: /params\nmetrics: [loss, lr]\nruntime:\n  image: x\n")
    res = CliRunner().invoke(train_command, ["-c", str(cfg), "--batch_per_device", "2", "--dry-run"])
    assert res.exit_code == 0, res.output
    plan = json.loads(res.output)
    assert plan["max_lr"] == 1e-4 and plan["batch_per_device"] == 2 and plan["nprocs"] == 4  # yaml, cli, yaml
    assert plan["grad_accum_steps"] == 1 and plan["metrics"] == ["loss", "lr"] and plan["parallel_mode"] == "fsdp"


def test_unknown_yaml_key_and_missing_required(tmp_path):
    cfg = tmp_path / "bad.yaml"
    cfg.write_text("nonsense: 1\n")
    res = CliRunner().invoke(train_command, ["-c", str(cfg), "--dry-run"])
    assert res.exit_code != 0 and "unknown option" in res.output
    res = CliRunner().invoke(train_command, ["--dry-run"])
    assert res.exit_code != 0 and "--train_type" in res.output


def test_step_arithmetic_and_scheduler_kwargs():
    assert compute_total_steps(1000, 4, 5, 2, 3) == (50 // 2) * 3
    o = dict(warmup_ratio=0.1, min_rate=None, schedule_type="wsd", stable_steps=None, decay_steps=None, cycle_length=None, t_mult=2)
    kw = scheduler_kwargs(o, 100)
    assert kw == {"warmup_steps": 10, "stable_steps": 72, "decay_steps": 18}


def test_runtime_exports(tmp_path):
    lines = runtime.exports("serve", {"runtime": {"image": "img:1", "gpus": [0, 1], "port": 8000}, "server": {"port": 1}})
    assert lines == ["export ASTRAI_IMAGE=img:1", "export ASTRAI_GPUS=0,1", "export ASTRAI_PORT=8000"]
    cfg = tmp_path / "s.yaml"
    cfg.write_text("runtime:\n  bogus: 1\n")
    assert runtime.main(["serve", str(cfg)]) == 1 and runtime.main(["x"]) == 2


def test_serve_load_generator_on_cpu():
    import torch

    from astrai_b200.cli.benchmark import _IdTokenizer, build_model, make_requests, run_serve
    from astrai_b200.inference import InferenceScheduler

    model = build_model("tiny", "cpu", torch.float32)
    sched = InferenceScheduler(model, _IdTokenizer(), max_batch_size=4, max_seq_len=512, page_size=16, kv_cache_tokens=4096, paged=True)
    reqs = make_requests(5, 100.0, 4096, 1, prompt_mean=48, prompt_range=(16, 96), prefix_len=32, out_range=(3, 6))
    assert all(reqs[i]["arrival"] < reqs[i + 1]["arrival"] for i in range(4))
    sched.start()
    try:
        res = run_serve(sched, reqs, 0.8, 0.95, 50)
    finally:
        sched.stop()
    assert res["completed"] == 5 and res["output_tokens"] >= 15 and res["ttft_ms_p50"] > 0 and res["tpot_ms_p50"] > 0


def test_benchmark_tool_takes_the_references_model_cache_and_backend_options(tmp_path):
    from astrai_b200.cli.benchmark import PRESETS, benchmark

    cfg = tmp_path / "arch.json"
    cfg.write_text(json.dumps({**PRESETS["tiny"], "num_hidden_layers": 1, "rms_norm_eps": 1e-6, "tie_word_embeddings": True, "rope_theta": 10000.0}))
    res = CliRunner().invoke(benchmark, ["prefill", "--config", str(cfg), "--device", "cpu", "--cache", "contiguous", "--backend", "torch_native",
                                         "--batch_size", "2", "--prompt_len", "24", "--trials", "1"])
    assert res.exit_code == 0, (res.output, res.exception)
    row = json.loads(res.output.strip().splitlines()[-1])
    assert row["benchmark"] == "prefill" and row["model"] == "arch.json" and row["cache"] == "contiguous" and row["backend"] == "torch_native"
    assert row["tok_per_s"] > 0

    res = CliRunner().invoke(benchmark, ["decode", "--preset", "tiny", "--device", "cpu", "--dtype", "float32", "--compare", "--batch_size", "2",
                                         "--prompt_len", "8", "--gen_len", "4"])
    assert res.exit_code == 0, (res.output, res.exception)
    lines = [json.loads(line) for line in res.output.strip().splitlines()]
    assert [r.get("benchmark") for r in lines] == ["decode", "decode", None] and lines[0]["cache"] == "paged"
    assert "compare" in lines[2] and any("_over_" in k for k in lines[2])
    assert lines[0]["cuda_graph"] is False  # a CPU model captures nothing

    from astrai_b200.config import AutoRegressiveLMConfig
    from astrai_b200.models import AutoRegressiveLM

    model_dir = tmp_path / "model"
    AutoRegressiveLM(AutoRegressiveLMConfig.from_file(cfg)).save_pretrained(str(model_dir))
    res = CliRunner().invoke(benchmark, ["decode", "--ckpt", str(model_dir), "--device", "cpu", "--batch_size", "1", "--prompt_len", "4", "--gen_len", "2"])
    assert res.exit_code == 0, (res.output, res.exception)
    assert json.loads(res.output.strip().splitlines()[-1])["model"] == "model"
