"""Pipeline parallelism: layer split, 1F1B order, and a multi-process CPU run against the whole model."""

import json
import os
import subprocess
import sys

import pytest

from astrai_b200.parallel.pipeline import schedule_1f1b, split_layers

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_split_layers_is_contiguous_and_even():
    assert split_layers(24, 4) == [0, 6, 12, 18, 24]
    assert split_layers(5, 2) == [0, 3, 5]
    assert split_layers(3, 3) == [0, 1, 2, 3]
    with pytest.raises(ValueError):
        split_layers(2, 3)


@pytest.mark.parametrize("stages,micro", [(1, 3), (2, 4), (4, 8), (4, 2)])
def test_1f1b_schedule_properties(stages, micro):
    for s in range(stages):
        steps = schedule_1f1b(stages, s, micro)
        assert [i for k, i in steps if k == "F"] == list(range(micro))
        assert [i for k, i in steps if k == "B"] == list(range(micro))
        alive = peak = 0
        done_f = set()
        for k, i in steps:
            if k == "F":
                done_f.add(i)
                alive += 1
            else:
                assert i in done_f  # a backward never precedes its forward
                alive -= 1
            peak = max(peak, alive)
        assert peak == min(stages - s, micro)  # activation memory bound of 1F1B


@pytest.mark.parametrize("stages,micro,moe,sft", [(4, 4, False, False), (2, 2, True, False), (3, 2, True, True)])
def test_pipeline_step_matches_whole_model(tmp_path, stages, micro, moe, sft):
    """Gradients and loss of one 1F1B window equal those of the whole model; with ``sft`` the batch holds packed documents
    with position ids and an uneven loss mask, and the whole model sees the batch in ONE piece (mean over trained tokens)."""
    out = str(tmp_path / "pp.json")
    from helpers import launch_ranks

    args = ["--out", out, "--micro", str(micro)] + (["--moe"] if moe else []) + (["--sft"] if sft else [])
    code, log = launch_ranks(stages, os.path.join(ROOT, "tests", "workers", "pp_compare.py"), args, 29720 + stages * 10 + micro + (5 if sft else 0),
                             env=dict(os.environ, OMP_NUM_THREADS="2"), cwd=ROOT)
    assert code == 0, log
    res = json.load(open(out))
    assert sum(r["n_keys"] for r in res) > 0
    for r in res:
        assert r["worst"] < 1e-4, r
        assert r["stray"] == [], r
    last = res[-1]
    assert abs(last["loss"] - last["ref_loss"]) < 1e-5
