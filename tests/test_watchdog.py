"""Rank-failure detection with store heartbeats: in-process over a HashStore, and across gloo ranks on the CPU."""

import json
import os
import subprocess
import sys
import time

import pytest
import torch.distributed as dist

from astrai_b200.parallel.watchdog import Heartbeat, RankFailure

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_missing_beats_and_announced_exit_are_detected():
    store = dist.HashStore()
    seen = []
    a = Heartbeat(0, 3, store=store, timeout_s=0.3, interval_s=0.05, on_failure=seen.extend).start()
    b = Heartbeat(1, 3, store=store, timeout_s=0.3, interval_s=0.05).start()
    c = Heartbeat(2, 3, store=store, timeout_s=0.3, interval_s=0.05).start()
    try:
        for step in range(1, 4):
            for h in (a, b, c):
                h.beat(step)
            time.sleep(0.05)
        a.check()  # everyone alive
        c.leave("done")  # an orderly exit is seen at the next scan, long before the timeout
        time.sleep(0.2)
        with pytest.raises(RankFailure) as exc:
            a.check()
        assert exc.value.ranks == [2] and "announced" in str(exc.value)
        b.stop()  # rank 1 goes silent: seen after the timeout
        deadline = time.time() + 3
        while 1 not in a.scan() and time.time() < deadline:
            a.beat()
            time.sleep(0.05)
        with pytest.raises(RankFailure) as exc:
            a.check()
        assert exc.value.ranks == [1, 2]
        while 1 not in seen and time.time() < deadline:
            time.sleep(0.01)  # the scanning thread records a dead rank first and calls on_failure right after
        assert sorted(seen) == [1, 2]
    finally:
        for h in (a, b, c):
            h.stop()


@pytest.mark.parametrize("mode", ["leave", "silent"])
def test_survivors_stop_between_steps_when_a_rank_goes_away(tmp_path, mode):
    out = str(tmp_path / "hb.json")
    from helpers import launch_ranks

    code, log = launch_ranks(3, os.path.join(ROOT, "tests", "workers", "heartbeat_ranks.py"), ["--out", out, "--victim", "1", "--mode", mode],
                             29790 if mode == "leave" else 29791, timeout=300, cwd=ROOT)
    assert code == 0, log
    res = {r: json.load(open(f"{out}.{r}")) for r in range(3)}
    assert res[1]["left_at"] == 4 and res[1]["steps"] == 3
    for r in (0, 2):
        assert res[r]["detected"] == [1], res  # found on the host, before the next collective was issued
        assert res[r]["steps"] == 3
        assert res[r]["seconds"] < (1.5 if mode == "leave" else 6.0)


@pytest.mark.parametrize("mode", ["fsdp", "ddp"])
def test_survivors_write_an_emergency_checkpoint_without_collectives(tmp_path, mode):
    """Three gloo ranks train through the real Trainer; rank 1 exits silently between steps.  The survivors must
    return within a bound (no barrier, no gather that waits for the dead rank) and leave the weights on disk."""
    out, ckpt = str(tmp_path / "res"), str(tmp_path / "ckpt")
    from helpers import launch_ranks

    code, log = launch_ranks(3, os.path.join(ROOT, "tests", "workers", "rank_loss_trainer.py"), ["--out", out, "--ckpt", ckpt, "--mode", mode],
                             29793 if mode == "fsdp" else 29794, timeout=300, cwd=ROOT)
    assert code == 0, log
    gone = float(open(out + ".gone").read())
    for r in (0, 2):
        res = json.load(open(f"{out}.{r}"))
        assert 1 in res["failure"], res
        assert res["returned_at"] - gone < 20.0, res  # heartbeat timeout 1.5 s + save; far below any process-group timeout
    dirs = [d for d in os.listdir(ckpt) if d.startswith("epoch_") and not d.endswith(".shards")]
    assert len(dirs) == 1
    root = os.path.join(ckpt, dirs[0])
    meta = json.load(open(os.path.join(root, "meta.json")))
    assert meta["emergency"] is True and 1 in meta["failed_ranks"]
    assert os.path.getsize(os.path.join(root, "model.safetensors")) > 0
    if mode == "fsdp":  # sharded optimizer state: one file per survivor, none gathered
        shards = sorted(os.listdir(root + ".shards"))
        assert shards == ["optimizer.rank0.pt", "optimizer.rank2.pt"]
        assert not os.path.exists(os.path.join(root, "optimizer.pt"))
    else:
        assert os.path.getsize(os.path.join(root, "optimizer.pt")) > 0
