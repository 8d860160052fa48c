"""Checkpoints on disk: layout, atomic replacement, completeness rules for restarts, model directories, sharded weights,
rank-0-reads-and-broadcasts loading (behaviours the reference checks in ``tests/data/test_checkpoint.py`` and relies on
in its restart scripts)."""

import json
import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _state():
    torch.manual_seed(0)
    return {"embed_tokens.weight": torch.randn(8, 4), "layers.0.mlp.up.weight": torch.randn(6, 4).bfloat16(), "norm.weight": torch.ones(4)}


def test_checkpoint_directory_layout_and_roundtrip(tmp_path):
    from astrai_b200.serialization import Checkpoint

    ck = Checkpoint(state_dict=_state(), epoch=3, consumed_samples=1200, config={"hidden_size": 4},
                    extra={"optimizer": {"step": 7, "m": torch.arange(3.0)}, "scheduler": {"last_epoch": 7}}, meta={"note": "hello"})
    ck.save(tmp_path / "epoch_3_step_7")
    names = sorted(p.name for p in (tmp_path / "epoch_3_step_7").iterdir())
    assert names == ["config.json", "meta.json", "model.safetensors", "optimizer.pt", "scheduler.pt"]
    assert not (tmp_path / "epoch_3_step_7.tmp").exists()
    meta = json.load(open(tmp_path / "epoch_3_step_7" / "meta.json"))
    assert meta["epoch"] == 3 and meta["consumed_samples"] == 1200 and meta["note"] == "hello" and "timestamp" in meta
    back = Checkpoint.load(tmp_path / "epoch_3_step_7")
    assert back.epoch == 3 and back.consumed_samples == 1200 and back.config == {"hidden_size": 4}
    assert back.extra["optimizer"]["step"] == 7 and torch.equal(back.extra["optimizer"]["m"], torch.arange(3.0))
    for k, v in _state().items():
        assert torch.equal(back.state_dict[k], v) and back.state_dict[k].dtype == v.dtype


def test_saving_again_replaces_files_and_keeps_what_others_wrote_there(tmp_path):
    from astrai_b200.serialization import Checkpoint

    d = tmp_path / "ck"
    Checkpoint(state_dict=_state(), epoch=1).save(d)
    (d / "metric.jsonl").write_text("{}\n")  # a file another component placed beside the checkpoint
    newer = {k: v + 1 for k, v in _state().items()}
    Checkpoint(state_dict=newer, epoch=2).save(d)
    back = Checkpoint.load(d)
    assert back.epoch == 2 and torch.equal(back.state_dict["norm.weight"], torch.full((4,), 2.0))
    assert (d / "metric.jsonl").read_text() == "{}\n"
    (tmp_path / "ck.tmp").mkdir()  # debris of a writer that died: the next save clears it
    (tmp_path / "ck.tmp" / "junk").write_text("x")
    Checkpoint(state_dict=_state(), epoch=3).save(d)
    assert Checkpoint.load(d).epoch == 3 and not (tmp_path / "ck.tmp").exists()


def test_only_complete_checkpoints_count_for_a_restart(tmp_path):
    from astrai_b200.serialization import Checkpoint
    from astrai_b200.serialization.checkpoint import is_complete, latest_complete

    extra = {"optimizer": {"step": 1}, "scheduler": {"last_epoch": 1}}
    assert latest_complete(tmp_path / "absent") is None and latest_complete(tmp_path) is None
    Checkpoint(state_dict=_state(), extra=extra).save(tmp_path / "epoch_0_step_10")
    Checkpoint(state_dict=_state(), extra=extra).save(tmp_path / "epoch_0_step_200")
    Checkpoint(state_dict=_state(), extra=extra).save(tmp_path / "epoch_1_step_30")
    Checkpoint(state_dict=_state()).save(tmp_path / "epoch_2_step_5")               # weights only: nothing to resume the optimizer from
    (tmp_path / "epoch_3_step_1").mkdir()                                           # an empty directory
    (tmp_path / "notes").mkdir()
    assert latest_complete(tmp_path).name == "epoch_1_step_30"                      # ordered by (epoch, step) as numbers, not as text
    (tmp_path / "epoch_1_step_30" / "optimizer.pt").write_bytes(b"")               # truncated by a crash
    assert not is_complete(tmp_path / "epoch_1_step_30") and latest_complete(tmp_path).name == "epoch_0_step_200"
    assert is_complete(tmp_path / "epoch_2_step_5", need=("meta.json", "model.safetensors"))


def test_load_any_understands_checkpoints_model_directories_and_sharded_weights(tmp_path):
    from safetensors.torch import save_file

    from astrai_b200.serialization import Checkpoint
    from astrai_b200.serialization.checkpoint import load_model_config, load_model_weights, save_model

    assert Checkpoint.load_any(tmp_path) is None
    save_model({"hidden_size": 4}, _state(), tmp_path / "model")
    plain = Checkpoint.load_any(tmp_path / "model")
    assert plain.epoch == 0 and plain.config == {"hidden_size": 4} and set(plain.state_dict) == set(_state())
    assert load_model_config(tmp_path / "model") == {"hidden_size": 4}
    sharded = tmp_path / "hf"
    sharded.mkdir()
    sd = {k: v.contiguous() for k, v in _state().items()}
    keys = sorted(sd)
    save_file({keys[0]: sd[keys[0]]}, str(sharded / "model-00001-of-00002.safetensors"))
    save_file({k: sd[k] for k in keys[1:]}, str(sharded / "model-00002-of-00002.safetensors"))
    index = {"weight_map": {keys[0]: "model-00001-of-00002.safetensors", **{k: "model-00002-of-00002.safetensors" for k in keys[1:]}}}
    (sharded / "model.safetensors.index.json").write_text(json.dumps(index))
    merged = load_model_weights(sharded)
    assert set(merged) == set(sd) and all(torch.equal(merged[k], sd[k]) for k in sd)
    assert set(Checkpoint.load_any(sharded).state_dict) == set(sd)
    with pytest.raises(FileNotFoundError):
        load_model_weights(tmp_path)


def test_non_contiguous_and_shared_tensors_are_written_as_independent_copies(tmp_path):
    from astrai_b200.serialization.checkpoint import load_safetensors, save_safetensors

    base = torch.arange(12.0).view(3, 4)
    sd = {"t": base.t(), "view": base[1], "again": base[1]}  # safetensors itself refuses shared or strided storage
    save_safetensors(sd, tmp_path / "w.safetensors")
    back = load_safetensors(tmp_path / "w.safetensors")
    assert torch.equal(back["t"], base.t()) and torch.equal(back["view"], base[1]) and torch.equal(back["again"], base[1])


def test_rank_zero_reads_and_every_rank_receives(tmp_path):
    from astrai_b200.serialization import Checkpoint

    ck = Checkpoint(state_dict=_state(), epoch=2, consumed_samples=64, config={"hidden_size": 4},
                    extra={"optimizer": {"step": 5, "m": torch.arange(4.0)}, "scheduler": {"last_epoch": 5}}, meta={"note": "shared"})
    ck.save(tmp_path / "ck")
    out = str(tmp_path / "res")
    from helpers import launch_ranks

    code, log = launch_ranks(3, os.path.join(ROOT, "tests", "workers", "ckpt_broadcast.py"), ["--ckpt", str(tmp_path / "ck"), "--out", out], 29788,
                             timeout=300, cwd=ROOT)
    assert code == 0, log
    got = [json.load(open(f"{out}.{r}")) for r in range(3)]
    want_sum = float(sum(v.double().sum() for v in _state().values()))
    for r, res in enumerate(got):
        assert res["rank"] == r and res["epoch"] == 2 and res["consumed"] == 64 and res["meta_note"] == "shared"
        assert res["keys"] == sorted(_state()) and res["sum"] == pytest.approx(want_sum) and res["bsd_sum"] == pytest.approx(want_sum)
        assert res["extra"] == ["optimizer", "scheduler"] and res["opt_step"] == 5 and res["config"] == {"hidden_size": 4}
        assert "torch.bfloat16" in res["dtypes"]  # dtypes survive the wire


def test_completeness_follows_the_checkpoints_own_file_list(tmp_path):
    """A run without a scheduler writes no scheduler.pt and can still be resumed; a checkpoint without optimizer state, or
    with one of its listed files missing or empty, cannot."""
    import os

    from astrai_b200.serialization import Checkpoint, is_complete, latest_complete

    weights = {"w": torch.ones(2, 2)}
    full = tmp_path / "epoch_0_step_1"
    Checkpoint(state_dict=weights, extra={"optimizer": {"state": {}}, "scheduler": {"last_epoch": 1}}, config={"a": 1}).save(full)
    no_sched = tmp_path / "epoch_0_step_2"
    Checkpoint(state_dict=weights, extra={"optimizer": {"state": {}}}, config={"a": 1}).save(no_sched)
    weights_only = tmp_path / "epoch_0_step_3"
    Checkpoint(state_dict=weights, config={"a": 1}).save(weights_only)
    assert is_complete(full) and is_complete(no_sched) and not is_complete(weights_only)
    assert latest_complete(tmp_path) == no_sched
    import json

    assert json.load(open(no_sched / "meta.json"))["files"] == ["config.json", "model.safetensors", "optimizer.pt"]
    os.truncate(no_sched / "optimizer.pt", 0)
    assert not is_complete(no_sched) and latest_complete(tmp_path) == full
    os.remove(full / "scheduler.pt")  # listed but gone
    assert not is_complete(full) and latest_complete(tmp_path) is None
    assert is_complete(weights_only, need=["meta.json", "model.safetensors"])  # an explicit list still decides alone
