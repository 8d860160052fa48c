"""Full-shard residency of the flat FSDP runtime (``reshard=True``) on gloo ranks: same training as the replicated
placement, and nothing whole at rest."""

import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(tmp_path, nproc, port, *extra):
    out = str(tmp_path / "res.json")
    from helpers import launch_ranks

    code, log = launch_ranks(nproc, os.path.join(ROOT, "tests", "workers", "fsdp_reshard.py"), ["--out", out, *extra], port, cwd=ROOT)
    assert code == 0, log
    return json.load(open(out))


@pytest.mark.parametrize("nproc,untied", [(2, False), (2, True), (3, False)])
def test_full_shard_placement_trains_like_the_replicated_one(tmp_path, nproc, untied):
    res = _run(tmp_path, nproc, 29730 + nproc + 10 * int(untied), *(["--untied"] if untied else []))
    assert res["keys"]
    # fp32 on the CPU: the two placements differ only in the order of the gradient sums
    assert res["a"] == pytest.approx(res["b"], abs=2e-5)
    assert res["a_norms"] == pytest.approx(res["b_norms"], rel=1e-4)
    assert res["a_eval"] == pytest.approx(res["b_eval"], abs=2e-5)
    assert res["max_weight_diff"] < 2e-5
    info = res["info"]
    assert info["at_rest_after_prepare"] == 0 and info["between_micro_batches"] == 0 and info["at_rest_after_save"] == 0
    assert info["whole_bytes"] > 0
    # never more than the current block, the prefetched one and the units outside the block list at the same time
    assert info["peak_units"] <= 2 + (info["units"] - 3)


def test_reshard_needs_library_collectives():
    from astrai_b200.parallel import ExecutorFactory

    with pytest.raises(ValueError, match="comm='nccl'"):
        ExecutorFactory.create("fsdp", comm="p2p", reshard=True)
