"""Trainer loop, callbacks, checkpoints, resume after an injected failure, strategies, distributed (gloo) paths."""

import json
import os
import signal
import subprocess
import sys
import textwrap

import pytest
import torch

from helpers import RandomTokens, tiny_config


def _model_tied():
    from astrai_b200.models import AutoRegressiveLM

    torch.manual_seed(0)
    return AutoRegressiveLM(tiny_config(tie_word_embeddings=True))


def _model_untied():
    from astrai_b200.models import AutoRegressiveLM

    torch.manual_seed(0)
    return AutoRegressiveLM(tiny_config())


def _fused_adamw(model):
    from astrai_b200.optim import FusedAdamW

    return FusedAdamW(model.parameters(), lr=1e-2)


def _torch_adamw(model):
    return torch.optim.AdamW(model.parameters(), lr=1e-2)


def _cosine(optimizer):
    from astrai_b200.trainer import SchedulerFactory

    return SchedulerFactory.create("cosine", optimizer, warmup_steps=1, lr_decay_steps=50)


def _train_config(tmp, dataset=None, **over):
    """Everything in the config is a module-level object so that spawned ranks can unpickle it."""
    from astrai_b200.config import TrainConfig

    base = dict(model_fn=_model_tied, strategy="seq", dataset=dataset or RandomTokens(40, 12),
                optimizer_fn=_fused_adamw, scheduler_fn=_cosine, batch_per_device=2, grad_accum_steps=2,
                ckpt_dir=str(tmp), ckpt_interval=2, device_type="cpu", backend="gloo", master_port=None)
    base.update(over)
    return TrainConfig(**base)


def test_train_writes_reference_layout(tmp_path):
    from astrai_b200.serialization import Checkpoint, is_complete
    from astrai_b200.trainer import Trainer

    Trainer(_train_config(tmp_path)).train()
    dirs = sorted(os.listdir(tmp_path))
    assert "epoch_0_step_10" in dirs and "epoch_0_step_2" in dirs
    last = tmp_path / "epoch_0_step_10"
    assert {"meta.json", "config.json", "model.safetensors", "optimizer.pt", "scheduler.pt", "metric.jsonl"} <= set(os.listdir(last))
    assert is_complete(last)
    ck = Checkpoint.load(last)
    assert ck.consumed_samples == 40 and ck.meta["strategy"] == "seq" and "embed_tokens.weight" in ck.state_dict
    rows = [json.loads(l) for l in open(last / "metric.jsonl")]
    steps = [r for r in rows if r["type"] == "step"]
    assert len(steps) == 10 and {"loss", "lr", "grad_norm"} <= set(steps[0])


def test_loss_goes_down_and_grad_accum_equivalence(tmp_path):
    from astrai_b200.trainer.train_context import TrainContextBuilder
    from astrai_b200.trainer import Trainer

    data = RandomTokens(4, 12)
    data.data = data.data[:1].repeat(4, 1)  # one sample repeated: the loss must fall
    cfg = _train_config(tmp_path, dataset=data, n_epoch=30, grad_accum_steps=1, ckpt_interval=10**6)
    tr = Trainer(cfg, callbacks=[])
    losses = []

    class Spy:
        def on_batch_end(self, ctx):
            losses.append(ctx.loss)

    tr.callbacks.append(Spy())
    tr.train()
    assert losses[-1] < losses[0] * 0.7


def test_resume_after_injected_failure(tmp_path):
    """The data source raises mid-epoch: an emergency checkpoint is written and a resumed run finishes the epoch."""
    from astrai_b200.serialization import Checkpoint, latest_complete
    from astrai_b200.trainer import Trainer

    with pytest.raises(RuntimeError, match="injected"):
        Trainer(_train_config(tmp_path, dataset=RandomTokens(40, 12, fail_after=12), ckpt_interval=100)).train()
    ck_dir = latest_complete(tmp_path)
    assert ck_dir is not None
    ck = Checkpoint.load(ck_dir)
    assert ck.consumed_samples == 12 and "optimizer" in ck.extra
    Trainer(_train_config(tmp_path, ckpt_interval=100)).train(param_path=str(ck_dir), resume=True)
    final = Checkpoint.load(latest_complete(tmp_path))
    assert final.consumed_samples == 40


def test_incomplete_checkpoint_is_skipped(tmp_path):
    from astrai_b200.serialization import latest_complete

    good = tmp_path / "epoch_0_step_2"
    bad = tmp_path / "epoch_0_step_4"
    for d in (good, bad):
        d.mkdir()
    for n in ("meta.json", "config.json", "model.safetensors", "optimizer.pt", "scheduler.pt"):
        (good / n).write_text("x")
    (bad / "meta.json").write_text("x")
    (bad / "model.safetensors").write_text("")  # truncated write
    assert latest_complete(tmp_path) == good


def test_gradient_checkpointing_matches_plain(tmp_path):
    from astrai_b200.models import AutoRegressiveLM
    from astrai_b200.models.decoder import DecoderBlock
    from astrai_b200.trainer import CallbackFactory

    torch.manual_seed(0)
    m = AutoRegressiveLM(tiny_config())
    ids = torch.randint(0, 1000, (2, 8))
    m(ids)["logits"].sum().backward()
    ref = {n: p.grad.clone() for n, p in m.named_parameters()}
    m.zero_grad()
    cb = CallbackFactory.create("gradient_checkpointing", modules=[DecoderBlock])

    class Ctx:
        model = m

    cb.on_train_begin(Ctx)
    m(ids)["logits"].sum().backward()
    cb.on_train_end(Ctx)
    for n, p in m.named_parameters():
        assert torch.allclose(p.grad, ref[n], atol=1e-6), n
    assert not hasattr(m.layers[0], "_plain_forward")


def test_strategies_losses_match_manual(tmp_path):
    from astrai_b200.models import AutoRegressiveLM
    from astrai_b200.trainer import StrategyFactory
    from astrai_b200.trainer.strategy import make_doc_boundary_mask

    torch.manual_seed(0)
    m = AutoRegressiveLM(tiny_config()).eval()
    ids = torch.randint(1, 1000, (2, 9))
    batch = {"input_ids": ids[:, :-1], "target_ids": ids[:, 1:]}
    out = StrategyFactory.create("seq", model=m, device="cpu", label_smoothing=0.1)(batch)
    ref = torch.nn.functional.cross_entropy(m(ids[:, :-1])["logits"].flatten(0, 1), ids[:, 1:].flatten(), label_smoothing=0.1)
    assert torch.allclose(out["loss"], ref, atol=1e-6) and out["metrics"]["loss"] == pytest.approx(ref.item(), rel=1e-5)
    pos = torch.tensor([[0, 1, 2, 0, 1, 2, 3, 0], [0, 1, 2, 3, 4, 5, 6, 7]])
    mask = make_doc_boundary_mask(pos)
    assert mask.shape == (2, 1, 8, 8) and not mask[0, 0, 3, 2] and mask[0, 0, 5, 3] and mask[1, 0, 7, 0]
    lm = torch.ones(2, 8, dtype=torch.bool)
    lm[:, :2] = False
    sft = StrategyFactory.create("sft", model=m, device="cpu")({**batch, "position_ids": pos, "loss_mask": lm})
    logits = m(ids[:, :-1], mask, position_ids=pos)["logits"]
    tgt = ids[:, 1:].masked_fill(~lm, -100)
    assert torch.allclose(sft["loss"], torch.nn.functional.cross_entropy(logits.flatten(0, 1), tgt.flatten(), ignore_index=-100), atol=1e-6)


def test_dpo_and_grpo_strategies():
    from astrai_b200.models import AutoRegressiveLM
    from astrai_b200.trainer import StrategyFactory

    torch.manual_seed(0)
    pol = AutoRegressiveLM(tiny_config())
    ref = AutoRegressiveLM(tiny_config()).eval()
    ref.load_state_dict(pol.state_dict())
    chosen = torch.randint(1, 1000, (2, 7))
    rejected = torch.randint(1, 1000, (2, 7))
    rejected[1, 5:] = 0
    mask = torch.ones(2, 7)
    mask[:, :3] = 0
    dpo = StrategyFactory.create("dpo", model=pol, device="cpu", ref_model=ref, beta=0.1)
    out = dpo({"chosen": chosen, "rejected": rejected, "chosen_mask": mask, "rejected_mask": mask})
    assert out["loss"].item() == pytest.approx(0.6931, abs=1e-3)  # identical policy and reference
    out["loss"].backward()

    class Ex:
        use_distributed = False

        def unwrap_model(self, m):
            return m.state_dict()

    old = AutoRegressiveLM(tiny_config()).eval()
    grpo = StrategyFactory.create("grpo", model=pol, device="cpu", old_model=old, ref_model=ref, executor=Ex(), group_size=2)
    grpo.sync_old_model()
    batch = {"prompts": torch.randint(1, 1000, (2, 4)), "responses": torch.randint(1, 1000, (2, 2, 5)),
             "masks": torch.ones(2, 2, 5, dtype=torch.bool), "rewards": torch.tensor([[1.0, 0.0], [0.5, 0.2]])}
    res = grpo(batch)
    assert set(res["metrics"]) >= {"policy_loss", "kl_loss", "loss"}
    assert abs(res["metrics"]["kl_loss"]) < 1e-6 and abs(res["metrics"]["policy_loss"]) < 1e-5  # ratio == 1, advantages sum to 0
    res["loss"].backward()


def test_moe_aux_loss_and_diagnostics_flow():
    from astrai_b200.models import AutoRegressiveLM
    from astrai_b200.trainer import StrategyFactory

    m = AutoRegressiveLM(tiny_config(ffn_type="moe", n_routed_experts=4, n_shared_experts=1, n_activated_experts=2)).train()
    ids = torch.randint(1, 1000, (2, 9))
    s = StrategyFactory.create("seq", model=m, device="cpu", moe_aux_loss_coef=0.5)
    out = s({"input_ids": ids[:, :-1], "target_ids": ids[:, 1:]})
    mt = out["metrics"]
    assert mt["moe_aux_loss_weighted"] == pytest.approx(0.5 * mt["moe_aux_loss"], rel=1e-5)
    assert mt["loss"] == pytest.approx(mt["task_loss"] + mt["moe_aux_loss_weighted"], rel=1e-5)
    assert {"router_entropy", "dead_expert_fraction", "load_imbalance_mean", "load_imbalance_max", "aux_loss"} <= set(s._moe_metrics)


def _two_rank_body(rank_tmp):
    """Runs inside each gloo rank: DDP(torch impl) training + broadcast helpers."""
    import torch.distributed as dist

    from astrai_b200.parallel import broadcast_state_dict, get_rank, get_world_size, only_on_rank
    from astrai_b200.trainer import Trainer

    assert get_world_size() == 2
    sd = {"a": torch.arange(4.0), "b": torch.ones(2, 2)} if get_rank() == 0 else None
    got = broadcast_state_dict(sd)
    assert torch.equal(got["a"], torch.arange(4.0))

    @only_on_rank(0, sync=True)
    def mark():
        open(os.path.join(rank_tmp, "rank0.txt"), "w").write("x")
        return 7

    assert mark() == (7 if get_rank() == 0 else None)
    t = torch.tensor([float(get_rank())])
    dist.all_reduce(t)
    assert t.item() == 1.0


def _ddp_train(tmp):
    from astrai_b200.trainer import Trainer

    Trainer(_train_config(tmp, parallel_mode="ddp", nprocs=2, ckpt_interval=10**6)).train()


def test_spawn_two_gloo_ranks(tmp_path):
    from astrai_b200.parallel import spawn_parallel_fn

    spawn_parallel_fn(_two_rank_body, world_size=2, backend="gloo", device_type="cpu", rank_tmp=str(tmp_path))
    assert (tmp_path / "rank0.txt").exists()


def test_ddp_two_ranks_cpu_training(tmp_path):
    from astrai_b200.serialization import Checkpoint, latest_complete
    from astrai_b200.trainer import Trainer

    Trainer(_train_config(tmp_path, parallel_mode="ddp", nprocs=2, ckpt_interval=10**6)).train()
    ck = Checkpoint.load(latest_complete(tmp_path))
    assert ck.consumed_samples == 40  # 40 samples over 2 ranks x batch 2


def test_fsdp_torch_impl_two_ranks_cpu(tmp_path):
    from astrai_b200.serialization import latest_complete
    from astrai_b200.trainer import Trainer

    # untied weights: FSDP2 shards the embedding and the head as separate groups
    cfg = _train_config(tmp_path, parallel_mode="fsdp", nprocs=2, ckpt_interval=10**6, optimizer_fn=_torch_adamw,
                        model_fn=_model_untied)
    Trainer(cfg).train()
    assert latest_complete(tmp_path) is not None


def test_attention_segments_equal_the_reference_masks():
    """Run boundaries built on the host describe the same relation as the reference's dense boolean masks."""
    from astrai_b200.ops.segments import from_position_ids, from_valid_mask
    from astrai_b200.trainer.strategy import causal_padding_mask, make_doc_boundary_mask

    pos = torch.tensor([[0, 1, 2, 0, 1, 0, 1, 2], [0, 1, 2, 3, 4, 5, 6, 7]])
    seg = from_position_ids(pos)
    assert seg.bounds == [0, 3, 5, 8, 16] and seg.max_len == 8 and seg.n_runs == 4
    assert torch.equal(seg.to_dense(), make_doc_boundary_mask(pos))
    short = seg.drop_last()
    assert short.seq_len == 7 and torch.equal(short.to_dense(), make_doc_boundary_mask(pos)[:, :, :-1, :-1])
    valid = torch.tensor([[0, 0, 1, 1, 1, 0], [1, 1, 1, 1, 1, 1]]).bool()
    seg = from_valid_mask(valid)
    dense, ref = seg.to_dense(), causal_padding_mask(valid)
    rows = valid[:, None, :, None].expand_as(ref)
    assert torch.equal(dense[rows], ref[rows])  # identical for every real query token (padding rows are never read)
    assert from_valid_mask(torch.tensor([[1, 0, 1]]).bool()) is None  # padding in the middle: no run form
