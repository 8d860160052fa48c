"""Host wrappers under deploy/: checkpoint listing / cleaning logic and command-line surface (no docker needed)."""

import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
COMPLETE = ("meta.json", "config.json", "model.safetensors", "optimizer.pt", "scheduler.pt")


def _sh(*args, env=None):
    return subprocess.run(["bash", *args], cwd=ROOT, capture_output=True, text=True, env={**os.environ, **(env or {})}, timeout=120)


@pytest.fixture
def job(tmp_path):
    ck = tmp_path / "ckpt"
    for name, files in (("epoch_0_step_10", COMPLETE), ("epoch_0_step_20", COMPLETE), ("epoch_1_step_5", COMPLETE),
                        ("epoch_1_step_30", COMPLETE[:-1])):  # the newest one lacks scheduler.pt: not resumable
        d = ck / name
        d.mkdir(parents=True)
        for f in files:
            (d / f).write_text("x")
    cfg = tmp_path / "train.yaml"
    cfg.write_text(f"runtime:\n  ckpt_dir: {ck}\n  container_name: test_job\n  auto_resume: true\n")
    return cfg, ck


def test_every_script_parses():
    for name in ("lib.sh", "train.sh", "serve.sh", "docker.sh", "pre_commit.sh", "train-entrypoint.sh"):
        assert _sh("-n", f"deploy/{name}").returncode == 0, name


def test_train_wrapper_lists_only_complete_checkpoints_in_order(job):
    cfg, ck = job
    out = _sh("deploy/train.sh", "list", str(cfg))
    assert out.returncode == 0, out.stderr
    assert [os.path.basename(p) for p in out.stdout.split()] == ["epoch_0_step_10", "epoch_0_step_20", "epoch_1_step_5"]
    latest = _sh("deploy/train.sh", "latest", str(cfg))
    assert latest.stdout.strip().endswith("epoch_1_step_5")


def test_clean_previews_then_deletes_and_keeps_the_newest(job):
    cfg, ck = job
    prev = _sh("deploy/train.sh", "clean", str(cfg), "--keep", "1")
    assert prev.returncode == 0 and "would remove" in prev.stdout and (ck / "epoch_0_step_10").exists()
    done = _sh("deploy/train.sh", "clean", str(cfg), "--keep", "1", "--force")
    assert done.returncode == 0, done.stderr
    assert not (ck / "epoch_0_step_10").exists() and not (ck / "epoch_0_step_20").exists()
    assert (ck / "epoch_1_step_5").exists() and (ck / "epoch_1_step_30").exists()  # incomplete ones are never touched


def test_unknown_runtime_keys_and_commands_are_refused(tmp_path):
    bad = tmp_path / "bad.yaml"
    bad.write_text("runtime:\n  no_such_key: 1\n")
    out = _sh("deploy/train.sh", "list", str(bad))
    assert out.returncode != 0 and "runtime" in out.stderr
    ok = tmp_path / "ok.yaml"
    ok.write_text("runtime: {}\n")
    assert _sh("deploy/train.sh", "frobnicate", str(ok)).returncode == 2
    assert "preflight" in _sh("deploy/serve.sh", "help").stdout and "clean" in _sh("deploy/train.sh", "help").stdout
