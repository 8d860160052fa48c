"""Preference (DPO) and policy-gradient (GRPO) training on two gloo ranks through the real Trainer: the frozen reference
and behaviour models every rank builds from the gathered weights, and what they hold after training (the reference's
``tests/parallel/test_broadcast_state_dict.py`` checks the same helpers)."""

import json
import os

import pytest
import torch

from helpers import tiny_config


def _model():
    from astrai_b200.models import AutoRegressiveLM

    torch.manual_seed(3)
    return AutoRegressiveLM(tiny_config(vocab_size=128, hidden_size=16, intermediate_size=32, max_position_embeddings=64))


def _adamw(model):
    return torch.optim.AdamW(model.parameters(), lr=5e-3)


class Pairs(torch.utils.data.Dataset):
    def __init__(self, n=16, seq=10):
        g = torch.Generator().manual_seed(1)
        self.chosen = torch.randint(3, 128, (n, seq), generator=g)
        self.rejected = torch.randint(3, 128, (n, seq), generator=g)
        self.rejected[:, :4] = self.chosen[:, :4]  # a shared prompt
        self.mask = torch.zeros(n, seq, dtype=torch.bool)
        self.mask[:, 4:] = True

    def __len__(self):
        return self.chosen.shape[0]

    def __getitem__(self, i):
        return {"chosen": self.chosen[i], "rejected": self.rejected[i], "chosen_mask": self.mask[i], "rejected_mask": self.mask[i]}


class Groups(torch.utils.data.Dataset):
    def __init__(self, n=16, prompt=5, group=3, resp=6):
        g = torch.Generator().manual_seed(2)
        self.prompts = torch.randint(3, 128, (n, prompt), generator=g)
        self.responses = torch.randint(3, 128, (n, group, resp), generator=g)
        self.rewards = torch.rand(n, group, generator=g)

    def __len__(self):
        return self.prompts.shape[0]

    def __getitem__(self, i):
        return {"prompts": self.prompts[i], "responses": self.responses[i], "masks": torch.ones_like(self.responses[i], dtype=torch.bool),
                "rewards": self.rewards[i]}


def _fingerprint(module_or_dict):
    sd = module_or_dict if isinstance(module_or_dict, dict) else module_or_dict.state_dict()
    return {k: float(v.detach().double().sum()) for k, v in sorted(sd.items())}


class Witness:
    """Writes, per rank, what the frozen copies and the policy hold when training starts and ends."""

    def __init__(self, out_dir):
        self.out_dir = out_dir
        self.begin = None

    def _state(self, context):
        s = context.strategy
        state = {"ref": _fingerprint(s.ref_model), "ref_trains": any(p.requires_grad for p in s.ref_model.parameters()),
                 "ref_mode": s.ref_model.training}
        if hasattr(s, "old_model"):
            state["old"] = _fingerprint(s.old_model)
        return state

    def on_train_begin(self, context):
        self.begin = self._state(context)

    def on_train_end(self, context):
        from astrai_b200.parallel import get_rank

        end = self._state(context)
        if hasattr(context.strategy, "sync_old_model"):
            context.strategy.sync_old_model()  # collective: every rank calls it
            end["old_synced"] = _fingerprint(context.strategy.old_model)
        policy = context.executor.unwrap_model(context.model)  # collective for sharded models; whole weights on rank 0
        end["policy"] = _fingerprint(policy) if policy is not None else None
        with open(os.path.join(self.out_dir, f"rank{get_rank()}.json"), "w") as fh:
            json.dump({"begin": self.begin, "end": end, "steps": context.optimizer_step}, fh)


def _run(tmp_path, strategy, mode, dataset, **strategy_kwargs):
    from astrai_b200.config import TrainConfig
    from astrai_b200.trainer import Trainer

    cfg = TrainConfig(model_fn=_model, strategy=strategy, dataset=dataset, optimizer_fn=_adamw, batch_per_device=2, grad_accum_steps=2,
                      ckpt_dir=str(tmp_path / "ck"), ckpt_interval=10**6, device_type="cpu", backend="gloo", master_port=None, nprocs=2,
                      parallel_mode=mode, strategy_kwargs=strategy_kwargs, metrics=["loss"])
    Trainer(cfg, callbacks=[Witness(str(tmp_path))]).train()
    return [json.load(open(tmp_path / f"rank{r}.json")) for r in range(2)]


def _close(a, b, tol=1e-9):
    return a.keys() == b.keys() and all(abs(a[k] - b[k]) <= tol * max(1.0, abs(a[k])) for k in a)


@pytest.mark.parametrize("mode", ["ddp", "fsdp"])
def test_dpo_reference_model_is_the_starting_policy_on_every_rank(tmp_path, mode):
    ranks = _run(tmp_path, "dpo", mode, Pairs(), beta=0.2)
    start = _fingerprint(_model())
    for r in ranks:
        assert r["steps"] == 2  # 16 pairs / (2 ranks x 2 per batch x 2 accumulation)
        assert _close(r["begin"]["ref"], start) and _close(r["end"]["ref"], start)  # whole (unsharded) and never trained
        assert r["begin"]["ref_trains"] is False and r["begin"]["ref_mode"] is False
    moved = ranks[0]["end"]["policy"]
    assert moved is not None and not _close(moved, start, tol=1e-6)  # while the policy did move


@pytest.mark.parametrize("mode", ["ddp", "fsdp"])
def test_grpo_behaviour_model_follows_the_policy_only_when_synced(tmp_path, mode):
    ranks = _run(tmp_path, "grpo", mode, Groups(), group_size=3, clip_eps=0.2, kl_coef=0.05)
    start = _fingerprint(_model())
    policy = ranks[0]["end"]["policy"]
    assert policy is not None and not _close(policy, start, tol=1e-6)
    for r in ranks:
        assert _close(r["begin"]["ref"], start) and _close(r["begin"]["old"], start)
        assert _close(r["end"]["ref"], start) and _close(r["end"]["old"], start)  # offline training never refreshes it
        assert _close(r["end"]["old_synced"], policy, tol=1e-6)  # the gathered policy, on every rank
