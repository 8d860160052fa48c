"""The model-parallel training modes (``parallel_mode = tp | cp | ep | pp``) through the real Trainer on gloo ranks (CPU).

Each mode trains a tiny decoder for three optimizer steps on the same global batches as a single process and must
reproduce its losses, gradient norms and - after gathering the shards - its final weights under the reference's
checkpoint keys and shapes.  Four ranks with blocks of two exercise the sub-groups (model-parallel x data-parallel).
"""

import json
import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
WORKER = os.path.join(ROOT, "tests", "workers", "mp_train.py")
_PORT = [29800]


def _run(tmp_path, name, nproc, *args):
    out, ckpt = str(tmp_path / f"{name}.json"), str(tmp_path / f"ck_{name}")
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="1")
    if nproc == 1:
        cmd = [sys.executable, WORKER, "--out", out, "--ckpt", ckpt, *args]
        for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "LOCAL_WORLD_SIZE"):
            env.pop(k, None)
        proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600, cwd=ROOT)
        assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-3000:]
    else:
        from helpers import launch_ranks

        _PORT[0] += 1
        code, log = launch_ranks(nproc, WORKER, ["--out", out, "--ckpt", ckpt, *args], _PORT[0], env=env, cwd=ROOT)
        assert code == 0, log
    return json.load(open(out))


def _same(run, ref):
    assert run["losses"] == pytest.approx(ref["losses"], abs=2e-5)
    assert run["norms"] == pytest.approx(ref["norms"], rel=1e-4)
    assert run["shapes"] == ref["shapes"]  # the gathered checkpoint has the unsharded keys and shapes
    for k, v in ref["sums"].items():
        assert run["sums"][k] == pytest.approx(v, rel=1e-4), k


@pytest.fixture(scope="module")
def dense_ref(tmp_path_factory):
    return _run(tmp_path_factory.mktemp("ref"), "ref", 1, "--mode", "none")


@pytest.fixture(scope="module")
def moe_ref(tmp_path_factory):
    return _run(tmp_path_factory.mktemp("refmoe"), "refmoe", 1, "--mode", "none", "--moe")


@pytest.mark.parametrize("mode,nproc,size", [("tp", 2, 0), ("cp", 2, 0), ("tp", 4, 2), ("cp", 4, 2)])
def test_dense_model_parallel_mode_matches_single_process(tmp_path, dense_ref, mode, nproc, size):
    _same(_run(tmp_path, mode, nproc, "--mode", mode, "--size", str(size)), dense_ref)


@pytest.mark.parametrize("nproc,size,extra", [(2, 0, []), (4, 2, ["--chunks", "2"])])
def test_pipeline_parallel_mode_matches_single_process(tmp_path, dense_ref, nproc, size, extra):
    """Two stages (one decoder layer each) on two ranks, two such pipelines on four; 1F1B over 2 or 4 pieces of the batch."""
    run = _run(tmp_path, "pp", nproc, "--mode", "pp", "--size", str(size), *extra)
    _same(run, dense_ref)
    assert run["optimizer_stages"] == 2  # the checkpoint carries the optimizer state of both stages


@pytest.fixture(scope="module")
def sft_ref(tmp_path_factory):
    return _run(tmp_path_factory.mktemp("refsft"), "refsft", 1, "--mode", "none", "--strategy", "sft", "--val", "--label_smoothing", "0.1")


@pytest.mark.parametrize("extra", [["--chunks", "4"]])
def test_pipeline_parallel_supervised_objective_and_validation(tmp_path, sft_ref, extra):
    """Packed documents with position ids and an uneven loss mask, label smoothing from the strategy's options, a held-out
    quarter scored after training: the pipeline's losses, norms, weights and validation loss are the single process's,
    whatever the number of pieces."""
    run = _run(tmp_path, "ppsft", 2, "--mode", "pp", "--strategy", "sft", "--val", "--label_smoothing", "0.1", *extra)
    _same(run, sft_ref)
    assert len(run["val"]) == 1 and run["val"] == pytest.approx(sft_ref["val"], abs=2e-5)


def test_tensor_parallel_supervised_objective_is_the_mean_over_all_trained_tokens(tmp_path, sft_ref):
    """The ranks of a tensor-parallel block hold slices of the batch's tokens with different numbers of trained tokens; the
    block's loss, gradients and validation loss must still be those of one process that sees the whole batch."""
    run = _run(tmp_path, "tpsft", 2, "--mode", "tp", "--strategy", "sft", "--val", "--label_smoothing", "0.1")
    _same(run, sft_ref)
    assert run["val"] == pytest.approx(sft_ref["val"], abs=2e-5)


@pytest.fixture(scope="module")
def sequence_refs(tmp_path_factory):
    """Single-process runs of the two sequence-level objectives, shared by the tensor- and pipeline-parallel comparisons."""
    root = tmp_path_factory.mktemp("refseq")
    return {s: _run(root, f"ref{s}", 1, "--mode", "none", "--strategy", s) for s in ("dpo", "grpo")}


@pytest.mark.parametrize("strategy", ["dpo", "grpo"])
def test_tensor_parallel_sequence_level_objectives_match_single_process(tmp_path, sequence_refs, strategy):
    """Preference pairs and scored response groups: every rank scores its token rows, the per-token log-probabilities are
    gathered over the block and every rank evaluates the same loss against whole frozen reference models."""
    run = _run(tmp_path, f"tp{strategy}", 2, "--mode", "tp", "--strategy", strategy)
    _same(run, sequence_refs[strategy])


def test_tensor_parallel_pads_sequence_level_batches_until_their_tokens_divide():
    from astrai_b200.parallel import ExecutorFactory
    from astrai_b200.parallel.mesh import ParallelMesh

    ex = ExecutorFactory.create("tp", grad_accum_steps=1, size=8)
    ex.mesh = ParallelMesh(world=8, rank=3, mp_size=8)
    pairs = {"chosen": torch.ones(3, 5, dtype=torch.long), "rejected": torch.ones(3, 5, dtype=torch.long),
             "chosen_mask": torch.ones(3, 5, dtype=torch.bool), "rejected_mask": torch.ones(3, 5, dtype=torch.bool)}
    out = ex.pad_sequences(pairs)
    assert out["chosen"].shape == (3, 8) and (6 * 8) % 8 == 0  # 6 rows: the first length from 5 up whose tokens divide by 8
    assert out["chosen"][:, 5:].eq(0).all() and not out["chosen_mask"][:, 5:].any() and out["chosen"][:, :5].eq(1).all()
    assert ex.shard_batch(out) is out  # whole sequences stay on every rank
    groups = {"prompts": torch.ones(2, 3, dtype=torch.long), "responses": torch.ones(2, 3, 4, dtype=torch.long),
              "masks": torch.ones(2, 3, 4, dtype=torch.bool), "rewards": torch.zeros(2, 3)}
    out = ex.pad_sequences(groups)
    assert out["responses"].shape == (2, 3, 5) and (6 * (3 + 5)) % 8 == 0 and not out["masks"][..., 4:].any()
    assert out["prompts"] is groups["prompts"] and out["rewards"] is groups["rewards"]
    even = {"chosen": torch.ones(4, 8, dtype=torch.long), "rejected": torch.ones(4, 8, dtype=torch.long),
            "chosen_mask": torch.ones(4, 8, dtype=torch.bool), "rejected_mask": torch.ones(4, 8, dtype=torch.bool)}
    assert ex.pad_sequences(even)["chosen"] is even["chosen"]  # nothing to do
    ex.mesh = ParallelMesh(world=1, rank=0, mp_size=1)
    assert ex.pad_sequences(pairs) is pairs


def test_gathered_row_values_are_the_identity_outside_a_group():
    from astrai_b200.parallel.tensor_parallel import gather_row_values

    v = torch.arange(4.0, requires_grad=True)
    assert gather_row_values(v) is v


@pytest.mark.parametrize("strategy,extra", [("dpo", ["--chunks", "4"]), ("grpo", [])])
def test_pipeline_parallel_sequence_level_objectives_match_single_process(tmp_path, sequence_refs, strategy, extra):
    """A piece of the 1F1B window holds whole preference pairs / whole response groups; the last stage scores them with
    whole frozen models and the pieces' losses add up to the batch's."""
    run = _run(tmp_path, f"pp{strategy}", 2, "--mode", "pp", "--strategy", strategy, *extra)
    _same(run, sequence_refs[strategy])


def test_pipeline_mode_is_refused_for_online_objectives(tmp_path):
    from astrai_b200.config import TrainConfig
    from astrai_b200.trainer.train_context import TrainContextBuilder

    cfg = TrainConfig(model_fn=lambda: None, strategy="online_dpo", dataset=[0], optimizer_fn=lambda m: None, ckpt_dir=str(tmp_path),
                      parallel_mode="pp", pp_size=2, nprocs=2, device_type="cpu", backend="gloo", reward_model_fn=lambda: None)
    with pytest.raises(ValueError, match="on prepared data"):
        TrainContextBuilder(cfg)._executor()


def test_pipeline_executor_hands_each_stage_its_own_optimizer_state_and_refuses_other_objectives():
    from astrai_b200.parallel import ExecutorFactory
    from astrai_b200.parallel.mesh import ParallelMesh

    ex = ExecutorFactory.create("pp", grad_accum_steps=1, size=2)
    ex.mesh = ParallelMesh(world=4, rank=3, mp_size=2)  # second stage of the second pipeline
    assert ex.data_parallel_size == 2 and ex.data_parallel_rank == 1 and ex._averaging_scale() in (1.0, 0.5)
    saved = {"pipeline_stages": [{"stage": 0}, {"stage": 1}]}
    assert ex.unpack_optimizer_state(saved) == {"stage": 1}
    assert ex.unpack_optimizer_state({"plain": True}) == {"plain": True}  # a checkpoint of another mode passes through
    with pytest.raises(RuntimeError, match="3 pipeline stages"):
        ex.unpack_optimizer_state({"pipeline_stages": [1, 2, 3]})
    with pytest.raises(NotImplementedError, match="token cross-entropy"):
        ex.pipeline_step(None, {"texts": torch.zeros(1, 2)}, 1.0)


@pytest.mark.parametrize("nproc,size", [(2, 0), (4, 2)])
def test_expert_parallel_mode_matches_single_process(tmp_path, moe_ref, nproc, size):
    _same(_run(tmp_path, "ep", nproc, "--mode", "ep", "--moe", "--size", str(size)), moe_ref)


def test_mesh_sizes_and_registration():
    from astrai_b200.parallel import ExecutorFactory, data_parallel_size, model_parallel_size

    assert {"tp", "cp", "ep", "pp"} <= set(ExecutorFactory.list_registered())
    assert model_parallel_size("pp", 8, pp_size=4) == 4 and data_parallel_size("pp", 8, pp_size=4) == 2
    assert model_parallel_size("tp", 8, tp_size=1) == 8 and model_parallel_size("tp", 8, tp_size=4) == 4
    assert data_parallel_size("tp", 8, tp_size=4) == 2 and data_parallel_size("cp", 8, cp_size=8) == 1
    assert data_parallel_size("ep", 8, ep_size=8) == 8 and data_parallel_size("fsdp", 8) == 8


def test_tensor_parallel_cuts_token_level_batches_and_refuses_unknown_ones():
    from astrai_b200.parallel import ExecutorFactory
    from astrai_b200.parallel.mesh import ParallelMesh

    ex = ExecutorFactory.create("tp", grad_accum_steps=1, size=2)
    ex.mesh = ParallelMesh(world=2, rank=0, mp_size=2)
    with pytest.raises(NotImplementedError):
        ex.shard_batch({"texts": torch.zeros(2, 4)})
    cut = ex.shard_batch({"input_ids": torch.zeros(2, 4, dtype=torch.long), "target_ids": torch.arange(8).view(2, 4)})
    assert cut["target_ids"].tolist() == [0, 1, 2, 3] and cut["input_ids"].shape == (2, 4)


def test_context_parallel_batch_is_cut_zigzag_with_global_positions():
    from astrai_b200.parallel import ExecutorFactory
    from astrai_b200.parallel.mesh import ParallelMesh

    ex = ExecutorFactory.create("cp", grad_accum_steps=1, size=2)
    ex.mesh = ParallelMesh(world=2, rank=1, mp_size=2)
    ids = torch.arange(16).view(2, 8)
    cut = ex.shard_batch({"input_ids": ids, "target_ids": ids + 1})
    assert cut["input_ids"].tolist() == [[2, 3, 4, 5], [10, 11, 12, 13]]  # chunks 1 and 2 of 4
    assert cut["position_ids"].tolist() == [[2, 3, 4, 5]] * 2
    with pytest.raises(NotImplementedError):
        ex.shard_batch({"input_ids": ids, "target_ids": ids, "position_ids": ids})


def test_capacity_limit_drops_only_the_overflow_and_keeps_every_rank_within_its_share():
    from astrai_b200.parallel.expert_parallel import limit_rows_per_rank

    torch.manual_seed(0)
    t, k, e, world = 64, 2, 8, 4                      # 128 pairs, 32 per destination when balanced
    idx = torch.randint(0, e, (t, k))
    idx[:40] = torch.tensor([0, 1])                   # 80 pairs pile up on rank 0 (experts 0 and 1)
    w = torch.rand(t, k, requires_grad=True)
    new_idx, new_w, counts, dropped = limit_rows_per_rank(idx, w, e, world, capacity_factor=1.5)
    cap = int(1.5 * t * k) // world                   # 48 rows of every receiver belong to this sender
    per_rank = counts.view(world, e // world).sum(1)
    assert int(counts.sum()) == t * k and int(per_rank.max()) <= cap
    kept = new_w != 0
    assert torch.equal(new_idx[kept], idx[kept]) and torch.equal(new_w[kept], w[kept].detach())  # kept pairs are untouched
    sent_to_0 = ((idx // 2) == 0)
    assert int(dropped) == int(sent_to_0.sum()) - cap == int((~kept).sum())
    flat_keep = kept.reshape(-1)[sent_to_0.reshape(-1)]
    assert flat_keep[:cap].all() and not flat_keep[cap:].any()                 # the first `cap` pairs in token order stay
    assert ((new_idx[~kept] // 2) != 0).all()                                   # the dropped ones were re-addressed elsewhere
    new_w.sum().backward()
    assert torch.equal(w.grad != 0, kept)                                       # dropped pairs get no gradient
    same_idx, same_w, same_counts, none = limit_rows_per_rank(idx, w.detach(), e, world, capacity_factor=4.0)
    assert torch.equal(same_idx, idx) and torch.equal(same_w, w.detach()) and int(none) == 0
    assert torch.equal(same_counts, torch.bincount(idx.reshape(-1), minlength=e).int())
    with pytest.raises(ValueError, match="at least 1"):
        limit_rows_per_rank(idx, w, e, world, capacity_factor=0.5)


def test_capacity_limit_places_every_pair_even_at_factor_one():
    from astrai_b200.parallel.expert_parallel import limit_rows_per_rank

    t, k, e, world = 32, 4, 8, 2
    idx = torch.zeros(t, k, dtype=torch.long)         # everything wants expert 0
    _, w, counts, dropped = limit_rows_per_rank(idx, torch.ones(t, k), e, world, capacity_factor=1.0)
    assert counts.view(world, -1).sum(1).tolist() == [64, 64] and int(dropped) == 64 and int((w == 0).sum()) == 64
