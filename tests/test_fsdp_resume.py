"""Sharded optimizer state survives save + resume on more than one rank (gloo ranks on the CPU)."""

import json
import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(tmp_path, port, *extra):
    out, ckpt = str(tmp_path / "res.json"), str(tmp_path / "ckpt")
    from helpers import launch_ranks

    code, log = launch_ranks(2, os.path.join(ROOT, "tests", "workers", "fsdp_resume.py"), ["--out", out, "--ckpt", ckpt, *extra], port, cwd=ROOT)
    assert code == 0, log
    return json.load(open(out))


@pytest.mark.parametrize("untied", [False, True])
def test_resumed_two_rank_run_matches_the_uninterrupted_one(tmp_path, untied):
    res = _run(tmp_path, 29720 + int(untied), *(["--untied"] if untied else []))
    assert res["layout"] == "full"  # every rank's shard was gathered into the one optimizer file
    assert res["a"] == pytest.approx(res["b"], abs=1e-6)  # steps 3 and 4 after the resume equal the uninterrupted run
    assert res["a_sum"] == pytest.approx(res["b_sum"], rel=1e-7)


def test_per_rank_shard_is_refused_by_another_rank():
    from astrai_b200.optim import FusedAdamW

    torch.manual_seed(0)
    model = torch.nn.Linear(16, 16, bias=False)
    opt = FusedAdamW(model.parameters(), lr=1e-2)
    # a shard written by rank 0 of 2 ...
    sd = opt.state_dict()
    sd.update(flat_units={"u": {"step": 3, "exp_avg": torch.zeros(8), "exp_avg_sq": torch.zeros(8), "master": None}},
              flat_sharded=True, flat_layout="shard", flat_rank=0, flat_world=2)
    opt.load_state_dict(sd)

    class Unit:
        name = "u"

    class Eng:
        rank, world_size = 1, 2

    opt._engine, opt._sharded = Eng(), True
    with pytest.raises(RuntimeError, match="shard 0 of 2"):  # ... must not be installed on rank 1
        opt._state_for(Unit(), torch.zeros(8))
