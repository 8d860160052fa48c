"""The host-side ``runtime:`` section of the YAML configs: flat keys and the reference's nested layout, with the
consistency rules the container wrappers rely on (behaviours the reference checks in ``tests/test_serve_runtime.py`` and
``tests/test_serve_cli.py``)."""

import pytest
import yaml
from click.testing import CliRunner

from astrai_b200.cli import runtime


def _write(tmp_path, doc, name="cfg.yaml"):
    path = tmp_path / name
    path.write_text(yaml.safe_dump(doc))
    return path


def _env(lines):
    return dict(line[len("export "):].split("=", 1) for line in lines)


# ------------------------------------------------------------------------------------------------------------ serve
def test_nested_serve_defaults(tmp_path):
    cfg = _write(tmp_path, {"runtime": {"paths": {"param": "./weights"}}, "server": {"device": "cuda"}})
    got = _env(runtime.exports("serve", yaml.safe_load(cfg.read_text()), cfg.parent))
    assert got["ASTRAI_PORT"] == "8000" and got["ASTRAI_PARAM_DIR"] == str((tmp_path / "weights").resolve())
    assert "ASTRAI_GPUS" not in got and "ASTRAI_CONTAINER" not in got  # all GPUs, no name: nothing to export


def test_nested_serve_single_device_port_and_name(tmp_path):
    doc = {"runtime": {"job_name": "chat-1", "port": 9001, "paths": {"param": "/srv/p"}, "gpu": {"devices": [3]},
                       "container": {"restart": "unless-stopped"}}, "server": {"port": 8000}}
    got = _env(runtime.exports("serve", doc, tmp_path))
    assert got == {"ASTRAI_CONTAINER": "chat-1", "ASTRAI_PORT": "9001", "ASTRAI_GPUS": "3", "ASTRAI_PARAM_DIR": "/srv/p",
                   "ASTRAI_RESTART": "unless-stopped"}


@pytest.mark.parametrize("doc,message", [
    ({"runtime": {"paths": {}, "gpu": {"devices": [0, 1]}}}, "single-device"),
    ({"runtime": {"paths": {}, "gpu": {"devices": []}}}, "non-empty list"),
    ({"runtime": {"paths": {}, "gpu": {"devices": ["a"]}}}, "non-negative integers"),
    ({"runtime": {"paths": {}, "gpu": {"enabled": False}}, "server": {"device": "cuda"}}, "must be 'cpu'"),
    ({"runtime": {"paths": {}, "gpu": {"enabled": False, "devices": [0]}}, "server": {"device": "cpu"}}, "ignored"),
    ({"runtime": {"paths": {}, "gpu": {"enabled": "yes"}}}, "boolean"),
    ({"runtime": {"paths": {}, "port": 70000}}, "between 1 and 65535"),
    ({"runtime": {"paths": {}, "port": 0}}, "between 1 and 65535"),
    ({"runtime": {"paths": {}, "port": "8000"}}, "integer"),
    ({"runtime": {"paths": {}, "port": True}}, "integer"),
    ({"runtime": {"paths": {}}, "server": {"port": 99999}}, "server.port"),
    ({"runtime": {"paths": {}, "job_name": "bad name"}}, "job_name"),
    ({"runtime": {"paths": "nope"}}, "mapping"),
    ({"runtime": {"paths": {}, "mystery": 1}}, "unknown runtime key"),
    ({"runtime": {"paths": {}, "environment": {"1BAD": "x"}}}, "environment name"),
    ({"runtime": {"paths": {}, "environment": {"OK": [1, 2]}}}, "scalar"),
])
def test_nested_serve_rejections(tmp_path, doc, message):
    with pytest.raises(ValueError, match=message):
        runtime.exports("serve", doc, tmp_path)


def test_serve_without_gpu_on_cpu(tmp_path):
    doc = {"runtime": {"paths": {"param": "/p"}, "gpu": {"enabled": False}}, "server": {"device": "cpu"}}
    assert _env(runtime.exports("serve", doc, tmp_path))["ASTRAI_GPUS"] == "none"


# ------------------------------------------------------------------------------------------------------------ train
TRAIN = {"job_name": "run_7", "paths": {"data": "data", "model": "/m", "checkpoints": "ck"}}


def test_nested_train_paths_devices_and_duration(tmp_path):
    doc = {"runtime": {**TRAIN, "gpu": {"devices": [0, 2, 5], "parallel_mode": "fsdp"}, "container": {"max_duration_hours": 1.5, "shm_size": "64g"}}}
    got = _env(runtime.exports("train", doc, tmp_path))
    assert got["ASTRAI_CONTAINER"] == "run_7" and got["ASTRAI_GPUS"] == "0,2,5" and got["ASTRAI_NPROCS"] == "3"
    assert got["ASTRAI_DATA_DIR"] == str((tmp_path / "data").resolve()) and got["ASTRAI_PARAM_DIR"] == "/m"
    assert got["ASTRAI_CKPT_DIR"] == str((tmp_path / "ck").resolve()) and got["ASTRAI_MAX_HOURS"] == "1.5" and got["ASTRAI_SHM_SIZE"] == "64g"
    all_gpus = _env(runtime.exports("train", {"runtime": TRAIN}, tmp_path))
    assert "ASTRAI_GPUS" not in all_gpus and "ASTRAI_MAX_HOURS" not in all_gpus


@pytest.mark.parametrize("gpu,message", [
    ({"devices": [0, 1], "parallel_mode": "none"}, "exactly one GPU"),
    ({"devices": [0], "parallel_mode": "ddp"}, "at least two"),
    ({"devices": [0], "parallel_mode": "tp"}, "at least two"),
    ({"devices": [1, 1]}, "duplicates"),
    ({"parallel_mode": "zero3"}, "parallel_mode must be one of"),
])
def test_nested_train_device_rules(tmp_path, gpu, message):
    with pytest.raises(ValueError, match=message):
        runtime.exports("train", {"runtime": {**TRAIN, "gpu": gpu}}, tmp_path)


def test_nested_train_needs_name_and_paths(tmp_path):
    with pytest.raises(ValueError, match="job_name"):
        runtime.exports("train", {"runtime": {"paths": TRAIN["paths"]}}, tmp_path)
    with pytest.raises(ValueError, match="paths.checkpoints"):
        runtime.exports("train", {"runtime": {"job_name": "a", "paths": {"data": "d", "model": "m"}}}, tmp_path)
    with pytest.raises(ValueError, match="must not be negative"):
        runtime.exports("train", {"runtime": {**TRAIN, "container": {"max_duration_hours": -1}}}, tmp_path)
    with pytest.raises(ValueError, match="must be a number"):
        runtime.exports("train", {"runtime": {**TRAIN, "container": {"max_duration_hours": "soon"}}}, tmp_path)


# ------------------------------------------------------------------------------------------------- flat + command
def test_flat_keys_still_work_and_are_checked(tmp_path):
    lines = runtime.exports("train", {"runtime": {"image": "img:2", "gpus": [0, 1], "auto_resume": True, "max_hours": 12, "nprocs": 2}})
    assert lines == ["export ASTRAI_IMAGE=img:2", "export ASTRAI_GPUS=0,1", "export ASTRAI_AUTO_RESUME=1", "export ASTRAI_MAX_HOURS=12",
                     "export ASTRAI_NPROCS=2"]
    with pytest.raises(ValueError, match="between 1 and 65535"):
        runtime.exports("serve", {"runtime": {"port": 123456}})
    with pytest.raises(ValueError, match="unknown runtime key"):
        runtime.exports("serve", {"runtime": {"data_dir": "/d"}})  # a training key
    assert runtime.exports("serve", {}) == [] and runtime.exports("train", {"runtime": None}) == []
    with pytest.raises(ValueError, match="mapping"):
        runtime.exports("train", {"runtime": [1]})
    assert runtime.exports("serve", {"runtime": {"image": "it's"}}) == ["export ASTRAI_IMAGE='it'\"'\"'s'"]  # shell-quoted


def test_command_line_exports_and_environment(tmp_path, capsys):
    cfg = _write(tmp_path, {"runtime": {**TRAIN, "environment": {"NCCL_DEBUG": "WARN", "OMP_NUM_THREADS": 8, "EMPTY": None}}})
    assert runtime.main(["train", str(cfg)]) == 0
    out = capsys.readouterr().out
    assert "export ASTRAI_CONTAINER=run_7" in out and "NCCL_DEBUG" not in out
    assert runtime.main(["train", str(cfg), "environment"]) == 0
    records = capsys.readouterr().out.split("\0")
    assert sorted(records[:3]) == ["EMPTY=", "NCCL_DEBUG=WARN", "OMP_NUM_THREADS=8"] and records[3] == ""  # yaml.safe_dump sorts keys
    assert runtime.main(["train", str(tmp_path / "missing.yaml")]) == 1
    assert runtime.main(["train", str(cfg), "bogus"]) == 2 and runtime.main(["deploy", str(cfg)]) == 2
    bad = _write(tmp_path, {"runtime": {**TRAIN, "gpu": {"devices": [0], "parallel_mode": "fsdp"}}}, "bad.yaml")
    assert runtime.main(["train", str(bad)]) == 1 and "at least two" in capsys.readouterr().err


# ------------------------------------------------------------------------------------------------------- serve CLI
def test_serve_command_merges_yaml_under_explicit_options(tmp_path, monkeypatch):
    import astrai_b200.inference as inference
    from astrai_b200.cli.serve import serve_command

    seen = {}
    monkeypatch.setattr(inference, "run_server", lambda **kw: seen.update(kw))
    cfg = _write(tmp_path, {"server": {"port": 9100, "max_batch_size": 64, "dtype": "float16", "chunked_prefill": True},
                            "runtime": {"paths": {"param": "./p"}}})
    res = CliRunner().invoke(serve_command, ["-c", str(cfg), "--max_batch_size", "8", "--param_path", str(tmp_path)])
    assert res.exit_code == 0, res.output
    import torch

    assert seen["port"] == 9100 and seen["max_batch_size"] == 8 and seen["dtype"] is torch.float16  # yaml, cli, yaml
    assert seen["chunked_prefill"] is True and seen["prefill_defer_steps"] == 8 and seen["page_size"] == 16


def test_serve_command_rejects_bad_values(tmp_path):
    from astrai_b200.cli.serve import serve_command

    bad = _write(tmp_path, {"server": {"dtype": "int4"}})
    res = CliRunner().invoke(serve_command, ["-c", str(bad)])
    assert res.exit_code != 0 and "dtype" in res.output
    res = CliRunner().invoke(serve_command, ["-c", str(tmp_path / "nowhere.yaml")])
    assert res.exit_code != 0
    unknown = _write(tmp_path, {"server": {"speed": "ludicrous"}}, "u.yaml")
    res = CliRunner().invoke(serve_command, ["-c", str(unknown)])
    assert res.exit_code != 0 and "unknown option" in res.output
