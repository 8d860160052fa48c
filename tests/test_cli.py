"""CLI surface: YAML precedence, dry-run plan, required options, runtime exports, step arithmetic."""

import json

import pytest

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


# ---- how the options become a training configuration -------------------------------------------------------------------------
def _options(tmp_path, *argv):
    """The merged option dictionary the command would train with (what --dry-run sees, before it is cut down to the plan)."""
    import click

    from astrai_b200.cli.common import flatten_sections, load_yaml, merge_config
    from astrai_b200.cli.train import SECTIONS

    ctx = train_command.make_context("train", list(argv))
    return merge_config(ctx, dict(ctx.params), flatten_sections(load_yaml(ctx.params.get("config")), SECTIONS))


def _tiny_run(tmp_path):
    import torch

    from astrai_b200.serialization import save_bin

    params, data = tmp_path / "params", tmp_path / "data"
    params.mkdir()
    (params / "config.json").write_text(json.dumps(dict(vocab_size=64, hidden_size=16, num_hidden_layers=2, num_attention_heads=2,
                                                        num_key_value_heads=1, intermediate_size=32, max_position_embeddings=16,
                                                        rms_norm_eps=1e-6, rope_theta=10000.0, tie_word_embeddings=False)))
    save_bin(str(data / "shard_0000"), {"sequence": [torch.arange(0, 64).repeat(20).int()]})
    return ["--train_type", "seq", "--data_root_path", str(data), "--param_path", str(params), "--device_type", "cpu"]


def test_optimizer_scheduler_and_strategy_options_reach_their_constructors(tmp_path):
    from astrai_b200.cli.train import optimizer_kwargs, scheduler_kwargs, strategy_kwargs

    base = _tiny_run(tmp_path)
    o = _options(tmp_path, *base, "--optimizer", "muon_adamw", "--muon_momentum", "0.9", "--no-muon_nesterov", "--muon_ns_steps", "3")
    assert optimizer_kwargs(o) == {"lr": 3e-4, "weight_decay": 0.1, "muon_momentum": 0.9, "muon_nesterov": False, "muon_ns_steps": 3,
                                   "muon_adjust_lr": "match_rms_adamw"}
    o = _options(tmp_path, *base, "--optimizer", "nora_nadamw", "--nora_lr", "0.01", "--max_lr", "1e-3")
    assert optimizer_kwargs(o) == {"lr": 1e-3, "weight_decay": 0.1, "nora_lr": 0.01, "nora_beta": 0.95, "nora_momentum": 0.95, "nora_weight_decay": 0.0}
    o = _options(tmp_path, *base, "--optimizer", "mano_adamw", "--no-mano_nesterov")
    assert optimizer_kwargs(o)["mano_nesterov"] is False and "muon_momentum" not in optimizer_kwargs(o)
    assert set(optimizer_kwargs(_options(tmp_path, *base, "--optimizer", "fused_adamw"))) == {"lr", "weight_decay"}

    o = _options(tmp_path, *base, "--schedule_type", "sgdr", "--t_mult", "3", "--min_rate", "0.2", "--warmup_ratio", "0.1")
    assert scheduler_kwargs(o, 200) == {"warmup_steps": 20, "min_rate": 0.2, "cycle_length": 180, "t_mult": 3}
    o = _options(tmp_path, *base, "--schedule_type", "sgdr", "--cycle_length", "40")
    assert scheduler_kwargs(o, 200)["cycle_length"] == 40
    o = _options(tmp_path, *base, "--schedule_type", "wsd", "--stable_steps", "50", "--decay_steps", "10", "--warmup_ratio", "0")
    assert scheduler_kwargs(o, 100) == {"warmup_steps": 0, "stable_steps": 50, "decay_steps": 10}
    assert scheduler_kwargs(_options(tmp_path, *base), 100) == {"warmup_steps": 5, "lr_decay_steps": 95}

    assert strategy_kwargs(_options(tmp_path, *base, "--label_smoothing", "0.1")) == {"label_smoothing": 0.1}
    assert strategy_kwargs(_options(tmp_path, *base[:1], "dpo", *base[2:], "--dpo_beta", "0.3")) == {"beta": 0.3}
    assert strategy_kwargs(_options(tmp_path, *base[:1], "online_grpo", *base[2:], "--group_size", "8", "--grpo_kl_coef", "0.05")) == {
        "clip_eps": 0.2, "kl_coef": 0.05, "group_size": 8}


@pytest.mark.parametrize("argv,expect", [
    (["--parallel_mode", "fsdp", "--fsdp_comm", "nvls"], {"comm": "nvls"}),
    (["--parallel_mode", "fsdp", "--fsdp_reshard"], {"comm": "nccl", "reshard": True, "impl": "flat"}),
    (["--parallel_mode", "tp", "--tp_size", "2", "--mp_comm", "nccl"], {"comm": "nccl"}),
    (["--parallel_mode", "ep"], {"comm": "p2p"}),
    (["--parallel_mode", "pp", "--pp_size", "2", "--pp_chunks", "4"], {"chunks": 4}),
    (["--parallel_mode", "cp", "--cp_size", "2", "--fsdp_comm", "nccl"], {"attn_comm": "p2p", "comm": "nccl"}),
    (["--parallel_mode", "ddp"], {}),
])
def test_parallel_options_become_executor_arguments(tmp_path, argv, expect):
    from astrai_b200.cli.train import build_train_config

    cfg, steps = build_train_config(_options(tmp_path, *_tiny_run(tmp_path), "--nprocs", "2", "--window_size", "16", "--batch_per_device", "2",
                                             "--grad_accum_steps", "2", "--n_epoch", "3", "--gradient_checkpointing", "--moe_aux_loss_coef", "0.05",
                                             "--no-persistent_workers", *argv))
    assert cfg.executor_kwargs == expect and cfg.parallel_mode == argv[1] and cfg.nprocs == 2
    assert cfg.moe_aux_loss_coef == 0.05 and cfg.persistent_workers is False and len(cfg.gradient_checkpointing_modules) == 1
    # 1280 tokens in windows of 16 -> 79 samples; ranks of one model-parallel block read the same samples
    readers = 1 if argv[1] in ("tp", "pp", "cp") else 2
    per_rank = -(-len(cfg.dataset) // readers)
    assert steps == max(-(-per_rank // 2) // 2, 1) * 3
    model = cfg.model_fn()
    assert model.config.hidden_size == 16 and next(model.parameters()).dtype.is_floating_point
    sched = cfg.scheduler_fn(cfg.optimizer_fn(model))
    assert sched.get_last_lr()[0] <= 3e-4
