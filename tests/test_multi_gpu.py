"""Multi-GPU tests (need >= 2 CUDA devices; each case runs as torchrun child processes on 127.0.0.1).

NVLS is switched off in NCCL for these runs and the fused kernels use plain peer loads / stores.
"""

import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _need_gpus(n):
    if not torch.cuda.is_available() or torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} GPUs")


def _torchrun(nproc, script, extra, port, timeout=420):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), script, *extra]
    proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=timeout, cwd=ROOT)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]


def test_fused_p2p_fsdp_matches_nccl_fsdp(tmp_path):
    _need_gpus(2)
    script = os.path.join(ROOT, "tests", "workers", "fsdp_compare.py")
    res = {}
    for i, comm in enumerate(("nccl", "p2p")):
        out = str(tmp_path / f"{comm}.json")
        _torchrun(2, script, ["--comm", comm, "--out", out], 29620 + i)
        res[comm] = json.load(open(out))
    a, b = res["nccl"], res["p2p"]
    assert b["status"] == 0
    for x, y in zip(a["losses"], b["losses"]):
        assert abs(x - y) < 2e-2, (a, b)
    for x, y in zip(a["norms"], b["norms"]):
        assert abs(x - y) / max(abs(x), 1e-6) < 2e-2, (a, b)
    assert abs(a["checksum"] - b["checksum"]) / a["checksum"] < 1e-3


def test_fused_tensor_parallel_mlp_matches_nccl(tmp_path):
    _need_gpus(2)
    out = str(tmp_path / "tp.json")
    _torchrun(2, os.path.join(ROOT, "tests", "workers", "tp_compare.py"), ["--out", out], 29640)
    for rank_res in json.load(open(out)):
        assert rank_res["status"] == 0
        for key in ("y", "dx", "d_gate_up", "d_down"):
            assert rank_res[key] < 3e-2, rank_res
        assert rank_res["y_vs_fp32"] < 5e-2, rank_res


def test_fused_context_parallel_attention_matches_nccl_and_fp32(tmp_path):
    _need_gpus(2)
    out = str(tmp_path / "cp.json")
    _torchrun(2, os.path.join(ROOT, "tests", "workers", "cp_compare.py"), ["--out", out], 29660)
    for rank_res in json.load(open(out)):
        assert rank_res["status"] == 0
        for key in ("out", "dq", "dk", "dv"):
            assert rank_res[key] < 2e-2, rank_res
            assert rank_res[key + "_vs_fp32"] < 4e-2, rank_res


def test_expert_parallel_moe_matches_single_gpu_experts(tmp_path):
    _need_gpus(2)
    out = str(tmp_path / "ep.json")
    _torchrun(2, os.path.join(ROOT, "tests", "workers", "ep_compare.py"), ["--out", out], 29680)
    for rank_res in json.load(open(out)):
        assert rank_res["status"] == 0
        for key in ("out", "dx", "d_gate_up", "d_down", "d_router"):
            assert rank_res[key] < 3e-2, rank_res


def test_sequence_sharded_model_step_matches_whole_sequence(tmp_path):
    _need_gpus(2)
    out = str(tmp_path / "cpm.json")
    _torchrun(2, os.path.join(ROOT, "tests", "workers", "cp_model.py"), ["--out", out], 29700)
    for r in json.load(open(out)):
        assert r["status"] == 0
        assert abs(r["loss_cp"] - r["loss_full"]) < 2e-2, r
        assert r["worst_grad"] < 5e-2, r


def test_fused_nvls_fsdp_matches_nccl_fsdp(tmp_path):
    """The multimem variants (in-switch reduction for the reduce-scatter, in-switch broadcast for the parameter gather);
    on a box without an NVSwitch multicast mapping the executor falls back to plain peer loads / stores."""
    _need_gpus(2)
    script = os.path.join(ROOT, "tests", "workers", "fsdp_compare.py")
    res = {}
    for i, comm in enumerate(("nccl", "nvls")):
        out = str(tmp_path / f"{comm}.json")
        _torchrun(2, script, ["--comm", comm, "--out", out], 29630 + i)
        res[comm] = json.load(open(out))
    a, b = res["nccl"], res["nvls"]
    assert b["status"] == 0
    for x, y in zip(a["losses"], b["losses"]):
        assert abs(x - y) < 2e-2, (a, b)
    for x, y in zip(a["norms"], b["norms"]):
        assert abs(x - y) / max(abs(x), 1e-6) < 2e-2, (a, b)
    assert abs(a["checksum"] - b["checksum"]) / a["checksum"] < 1e-3


@pytest.mark.parametrize("extra", [[], ["--untied"]])
def test_fused_fsdp_save_and_resume_matches_uninterrupted_run(tmp_path, extra):
    """Two GPUs, fused peer-memory FSDP: train, save (optimizer shards gathered), rebuild, load, train on; the losses
    of the steps after the resume and the final parameters must equal the uninterrupted run."""
    _need_gpus(2)
    out = str(tmp_path / "resume.json")
    _torchrun(2, os.path.join(ROOT, "tests", "workers", "fsdp_resume.py"),
              ["--out", out, "--ckpt", str(tmp_path / "ckpt"), "--device", "cuda", "--comm", "p2p", *extra], 29700 + len(extra))
    res = json.load(open(out))
    assert res["layout"] == "full"
    for x, y in zip(res["a"], res["b"]):
        assert abs(x - y) < 2e-2, res
    assert abs(res["a_sum"] - res["b_sum"]) / res["a_sum"] < 1e-3, res


def _mp_run(tmp_path, name, nproc, port, *args):
    out = str(tmp_path / f"{name}.json")
    script = os.path.join(ROOT, "tests", "workers", "mp_train.py")
    common = ["--out", out, "--ckpt", str(tmp_path / f"ck_{name}"), "--device", "cuda", "--dtype", "bfloat16", "--seq", "512",
              "--hidden", "256", "--bpd", "2", "--lr", "1e-3", *args]
    if nproc == 1:
        env = {k: v for k, v in os.environ.items() if k not in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "LOCAL_WORLD_SIZE")}
        proc = subprocess.run([sys.executable, script, *common], env=env, capture_output=True, text=True, timeout=420, cwd=ROOT)
        assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    else:
        _torchrun(nproc, script, common, port)
    return json.load(open(out))


@pytest.mark.parametrize("mode,moe", [("tp", False), ("cp", False), ("ep", True)])
def test_model_parallel_trainer_modes_fused_and_collective_arms(tmp_path, mode, moe):
    """parallel_mode tp / cp / ep through the real Trainer on 2 GPUs in bf16: the fused peer-memory arm and the NCCL arm
    must both reproduce the single-GPU run (losses, gradient norms, gathered weights with the unsharded keys)."""
    _need_gpus(2)
    extra = ["--moe"] if moe else []
    ref = _mp_run(tmp_path, "ref", 1, 0, "--mode", "none", *extra)
    base = {"tp": 29720, "cp": 29730, "ep": 29740}[mode]
    for i, comm in enumerate(("nccl", "p2p")):
        run = _mp_run(tmp_path, f"{mode}_{comm}", 2, base + i, "--mode", mode, "--comm", comm, *extra)
        assert run["shapes"] == ref["shapes"], comm
        for a, b in zip(run["losses"], ref["losses"]):
            assert abs(a - b) < 3e-2, (comm, run["losses"], ref["losses"])
        for a, b in zip(run["norms"], ref["norms"]):
            assert abs(a - b) / max(abs(b), 1e-6) < 5e-2, (comm, run["norms"], ref["norms"])
        for k, v in ref["sums"].items():
            assert abs(run["sums"][k] - v) / max(v, 1e-6) < 2e-2, (comm, k)


def test_pipeline_parallel_trainer_mode_matches_single_gpu(tmp_path):
    """parallel_mode pp through the real Trainer on 2 GPUs in bf16 (two stages, 1F1B over two pieces, NCCL point-to-point
    messages, gradients in the flat runtime's fp32 buffers): losses, norms and gathered weights of the single-GPU run."""
    _need_gpus(2)
    ref = _mp_run(tmp_path, "ref", 1, 0, "--mode", "none")
    run = _mp_run(tmp_path, "pp", 2, 29760, "--mode", "pp")
    assert run["shapes"] == ref["shapes"] and run["optimizer_stages"] == 2
    for a, b in zip(run["losses"], ref["losses"]):
        assert abs(a - b) < 3e-2, (run["losses"], ref["losses"])
    for a, b in zip(run["norms"], ref["norms"]):
        assert abs(a - b) / max(abs(b), 1e-6) < 5e-2, (run["norms"], ref["norms"])
    for k, v in ref["sums"].items():
        assert abs(run["sums"][k] - v) / max(v, 1e-6) < 2e-2, k


def test_tensor_parallel_serving_on_two_gpus(tmp_path):
    """One serving replica over 2 GPUs in bf16 with CUDA-graph decode (the all-reduces of the cut blocks are inside the
    graphs): every request finishes, and the greedy streams start like the single-GPU ones (bf16 sums in another order
    may flip a near-tie later on)."""
    _need_gpus(2)
    out = str(tmp_path / "tp_serve.json")
    _torchrun(2, os.path.join(ROOT, "tests", "workers", "tp_serve.py"), ["--out", out, "--device", "cuda"], 29765, timeout=150)
    res = json.load(open(out))
    assert res["finished"] and res["local_heads"] == 2 and res["pool_heads"] == 1 and res["sampled_pieces"] == 6
    same_start = sum(g.split(">")[:2] == w.split(">")[:2] for g, w in zip(res["got"], res["want"]))
    assert same_start >= 4, res
    assert all(g.count("<") == w.count("<") for g, w in zip(res["got"], res["want"]))


def test_full_shard_fsdp_matches_replicated_fsdp(tmp_path):
    """``reshard=True`` on 2 GPUs (bf16, NCCL gathers / reduce-scatters on the side stream, storages released and
    re-created around every unit): same losses, norms and weights as the replicated placement, nothing whole at rest."""
    _need_gpus(2)
    out = str(tmp_path / "reshard.json")
    _torchrun(2, os.path.join(ROOT, "tests", "workers", "fsdp_reshard.py"), ["--out", out, "--device", "cuda", "--layers", "4"], 29690)
    res = json.load(open(out))
    for x, y in zip(res["a"], res["b"]):
        assert abs(x - y) < 2e-2, res
    for x, y in zip(res["a_norms"], res["b_norms"]):
        assert abs(x - y) / max(abs(x), 1e-6) < 2e-2, res
    assert abs(res["a_eval"] - res["b_eval"]) < 2e-2
    assert res["max_weight_diff"] < 2e-2
    info = res["info"]
    assert info["at_rest_after_prepare"] == 0 and info["between_micro_batches"] == 0 and info["at_rest_after_save"] == 0
    assert info["peak_units"] <= 2 + (info["units"] - 4)
