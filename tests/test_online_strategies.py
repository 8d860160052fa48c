"""GRPO / DPO objectives, their online (rollout-driven) mode and the rollout runner with a real tiny model and the real
scheduler on the CPU (behaviours the reference checks in ``tests/trainer/test_grpo_strategy.py``,
``test_online_strategy.py``, ``test_rollout.py`` and ``test_loss_output.py``)."""

import copy

import pytest
import torch

from helpers import build_tokenizer_dir, tiny_config


@pytest.fixture(scope="module")
def tok(tmp_path_factory):
    from astrai_b200.tokenize import AutoTokenizer

    return AutoTokenizer.from_pretrained(build_tokenizer_dir(str(tmp_path_factory.mktemp("tok"))))


def _model(seed=0, **over):
    from astrai_b200.models import AutoRegressiveLM

    torch.manual_seed(seed)
    return AutoRegressiveLM(tiny_config(vocab_size=512, hidden_size=32, intermediate_size=64, max_position_embeddings=128, **over))


class _Exec:
    """The two executor calls the strategies use."""

    use_distributed = False

    def unwrap_model(self, model):
        return model.state_dict()


def _grpo(model=None, **kw):
    from astrai_b200.trainer import StrategyFactory

    model = model or _model()
    old, ref = copy.deepcopy(model).requires_grad_(False), copy.deepcopy(model).requires_grad_(False)
    return StrategyFactory.create("grpo", model=model, device="cpu", old_model=old, ref_model=ref, executor=_Exec(), **kw)


def _grpo_batch(b=2, g=3, p=5, r=6, seed=0):
    gen = torch.Generator().manual_seed(seed)
    prompts = torch.randint(3, 500, (b, p), generator=gen)
    prompts[0, :2] = 0  # left padding
    responses = torch.randint(3, 500, (b, g, r), generator=gen)
    masks = torch.ones(b, g, r, dtype=torch.bool)
    masks[0, 1, 4:] = False
    masks[1, 2, 2:] = False
    responses = responses * masks
    rewards = torch.tensor([[1.0, 0.0, 0.5], [0.2, 0.9, 0.1]])[:b, :g]
    return {"prompts": prompts, "prompt_mask": prompts.ne(0), "responses": responses, "masks": masks, "rewards": rewards}


# ------------------------------------------------------------------------------------------------------------ GRPO
def test_grpo_loss_is_finite_and_reports_its_parts():
    s = _grpo()
    out = s(_grpo_batch())
    assert torch.isfinite(out["loss"]) and out["loss"].requires_grad
    m = out["metrics"].resolved()
    assert {"policy_loss", "kl_loss", "loss"} <= set(m)
    assert m["loss"] == pytest.approx(m["policy_loss"] + m["kl_loss"], abs=1e-6)
    assert m["kl_loss"] == pytest.approx(0.0, abs=1e-6)  # policy == reference at the start: the KL term vanishes


def test_grpo_backward_reaches_the_policy_only():
    s = _grpo()
    s(_grpo_batch())["loss"].backward()
    assert any(p.grad is not None and p.grad.abs().sum() > 0 for p in s.model.parameters())
    assert all(p.grad is None for p in s.old_model.parameters()) and all(p.grad is None for p in s.ref_model.parameters())


def test_grpo_identical_rewards_give_zero_policy_gradient():
    s = _grpo()
    batch = _grpo_batch()
    batch["rewards"] = torch.full_like(batch["rewards"], 0.7)
    out = s(batch)
    assert out["metrics"].resolved()["policy_loss"] == pytest.approx(0.0, abs=1e-6)  # no advantage without spread
    out["loss"].backward()
    total = sum(float(p.grad.abs().sum()) for p in s.model.parameters() if p.grad is not None)
    assert total < 1e-5


def test_grpo_ignores_prompt_and_padding_tokens():
    """Changing masked response positions, or the content of left padding, changes nothing."""
    s = _grpo()
    batch = _grpo_batch()
    base = float(s(batch)["loss"].detach())
    changed = {k: v.clone() for k, v in batch.items()}
    changed["responses"][0, 1, 4:] = 77   # behind the response's end
    changed["responses"][1, 2, 2:] = 99
    assert float(s(changed)["loss"].detach()) == pytest.approx(base, abs=1e-6)
    moved = {k: v.clone() for k, v in batch.items()}
    moved["rewards"] = batch["rewards"] * 3.0 + 5.0  # advantages are standardised per group
    assert float(s(moved)["loss"].detach()) == pytest.approx(base, abs=1e-5)


def test_grpo_clipping_bounds_the_surrogate():
    """With an old policy far from the current one the clipped objective differs from the unclipped one."""
    model = _model()
    s = _grpo(model, clip_eps=0.2)
    with torch.no_grad():
        for p in s.old_model.parameters():
            p.add_(0.3 * torch.randn_like(p))
    wide = _grpo(model, clip_eps=1e6)
    wide.old_model.load_state_dict(s.old_model.state_dict())
    batch = _grpo_batch()
    a, b = float(s(batch)["metrics"].resolved()["policy_loss"]), float(wide(batch)["metrics"].resolved()["policy_loss"])
    assert a != pytest.approx(b, abs=1e-6) and a >= b - 1e-6  # min(unclipped, clipped) can only lower the objective = raise the loss


def test_grpo_sync_old_model_copies_the_policy():
    s = _grpo()
    with torch.no_grad():
        for p in s.model.parameters():
            p.add_(0.1)
    assert any(not torch.equal(a, b) for a, b in zip(s.model.state_dict().values(), s.old_model.state_dict().values()))
    s.sync_old_model()
    assert all(torch.equal(a, b) for a, b in zip(s.model.state_dict().values(), s.old_model.state_dict().values()))
    assert all(not p.requires_grad for p in s.old_model.parameters())


# ------------------------------------------------------------------------------------------------------------- DPO
def _dpo(model=None, **kw):
    from astrai_b200.trainer import StrategyFactory

    model = model or _model()
    ref = copy.deepcopy(model).requires_grad_(False)
    return StrategyFactory.create("dpo", model=model, device="cpu", ref_model=ref, executor=_Exec(), **kw)


def _dpo_batch(seed=0):
    gen = torch.Generator().manual_seed(seed)
    chosen, rejected = torch.randint(3, 500, (2, 9), generator=gen), torch.randint(3, 500, (2, 9), generator=gen)
    rejected[:, :4] = chosen[:, :4]  # shared prompt
    chosen[1, 7:] = 0
    cm = torch.zeros(2, 9, dtype=torch.bool)
    cm[:, 4:] = True
    cm[1, 7:] = False
    rm = torch.zeros(2, 9, dtype=torch.bool)
    rm[:, 4:] = True
    return {"chosen": chosen, "rejected": rejected, "chosen_mask": cm, "rejected_mask": rm}


def test_dpo_starts_at_log_two_and_is_differentiable():
    s = _dpo()
    out = s(_dpo_batch())
    assert float(out["loss"]) == pytest.approx(0.6931, abs=1e-3)  # policy == reference: margin 0
    out["loss"].backward()
    assert any(p.grad is not None and p.grad.abs().sum() > 0 for p in s.model.parameters())
    assert all(p.grad is None for p in s.ref_model.parameters())


def test_dpo_prefers_the_chosen_answer_after_a_few_steps():
    s = _dpo(beta=0.5)
    opt = torch.optim.SGD(s.model.parameters(), lr=0.5)
    batch = _dpo_batch()
    first = float(s(batch)["loss"])
    for _ in range(5):
        opt.zero_grad()
        s(batch)["loss"].backward()
        opt.step()
    assert float(s(batch)["loss"]) < first
    before = [p.clone() for p in s.ref_model.parameters()]
    assert all(torch.equal(a, b) for a, b in zip(before, s.ref_model.parameters()))  # the reference never moves


def test_dpo_reduction_modes_differ_only_by_length_normalisation():
    model = _model()
    a, b = _dpo(model, reduction="sum"), _dpo(model, reduction="mean")
    batch = _dpo_batch()
    with torch.no_grad():
        for p in model.parameters():
            p.add_(0.05 * torch.randn_like(p))  # move the policy off the reference so that the margin is not 0
    assert float(a(batch)["loss"]) != pytest.approx(float(b(batch)["loss"]), abs=1e-7)


# ---------------------------------------------------------------------------------------------------------- online
class _Reward:
    def __init__(self, values=None):
        self.values, self.calls = values, 0

    def score(self, prompts, responses):
        self.calls += 1
        if self.values is not None:
            return self.values
        return torch.tensor([[float(len(r)) + 0.1 * j for j, r in enumerate(row)] for row in responses])


def _runner(tok, model, group=3, interval=2, reward=None, max_tokens=5):
    from astrai_b200.inference import InferenceScheduler
    from astrai_b200.trainer.rollout import BaseRewardModel, RolloutGenerator, RolloutRunner

    BaseRewardModel.register(_Reward)
    sched = InferenceScheduler(model, tok, max_batch_size=8, max_seq_len=96, enable_cuda_graph=False)
    gen = RolloutGenerator(sched, tok, max_tokens=max_tokens, group_size=group, temperature=1.0)
    return RolloutRunner(gen, reward or _Reward(), rollout_interval=interval), sched


BATCH = {"messages": [[{"role": "user", "content": "hello"}], [{"role": "system", "content": "be brief"}, {"role": "user", "content": "hi there"}]]}


def test_factory_knows_the_online_names_and_the_base_strategy_declines():
    from astrai_b200.trainer import StrategyFactory
    from astrai_b200.trainer.strategy import BaseStrategy, DPOStrategy, GRPOStrategy

    assert StrategyFactory._entries["online_grpo"] is GRPOStrategy and StrategyFactory._entries["online_dpo"] is DPOStrategy
    base = BaseStrategy(torch.nn.Linear(2, 2), "cpu")
    assert not base.supports_online()
    with pytest.raises(NotImplementedError, match="online rollout"):
        base.prepare_from_rollout(None)
    assert _grpo().supports_online() and _dpo().supports_online()


def test_rollout_generator_shapes_masks_and_logprobs(tok):
    model = _model().train()
    runner, _ = _runner(tok, model, group=3)
    raw = runner.generator.generate(BATCH)
    assert model.training  # generation ran in eval mode and restored the flag
    b, g, r = raw.responses.shape
    assert (b, g) == (2, 3) and 1 <= r <= 5
    assert raw.prompts.shape == raw.prompt_mask.shape and raw.prompt_mask[:, -1].all()  # left padded
    assert (raw.responses[~raw.response_mask] == 0).all() and (raw.logprobs_old[~raw.response_mask] == 0).all()
    assert (raw.logprobs_old[raw.response_mask] <= 0).all()
    assert len(raw.prompt_texts) == 2 and [len(x) for x in raw.response_texts] == [3, 3]
    assert raw.prompt_texts[1].count("be brief") == 1


def test_rollout_logprobs_are_the_policys_own(tok):
    """The behaviour log-probabilities returned with a rollout equal the model's log-probabilities of those tokens."""
    from astrai_b200.trainer.strategy import get_logprobs, padded_causal_attention

    model = _model().eval()
    runner, _ = _runner(tok, model, group=2, max_tokens=4)
    raw = runner.generator.generate({"messages": BATCH["messages"][:1]})
    p = raw.prompts[0][raw.prompt_mask[0]]
    for j in range(2):
        n = int(raw.response_mask[0, j].sum())
        seq = torch.cat([p, raw.responses[0, j, :n]])[None]
        loss_mask = torch.zeros_like(seq, dtype=torch.bool)
        loss_mask[0, len(p):] = True
        with torch.no_grad():
            lp = get_logprobs(model, seq, padded_causal_attention(seq.ne(-1)), loss_mask, "none")["logprobs"][0, len(p) - 1:]
        assert torch.allclose(lp[:n], raw.logprobs_old[0, j, :n], atol=1e-4)


def test_bad_rollout_batches_and_bad_rewards_are_refused(tok):
    runner, _ = _runner(tok, _model())
    with pytest.raises(ValueError, match="messages"):
        runner.generator.generate({"text": ["x"]})
    bad, _ = _runner(tok, _model(), reward=_Reward(torch.zeros(2, 5)))
    with pytest.raises(ValueError, match="expected"):
        bad(BATCH)


def test_runner_cache_interval_and_clear(tok):
    reward = _Reward()
    runner, _ = _runner(tok, _model(), interval=2, reward=reward)
    first, fresh = runner(BATCH)
    assert fresh and reward.calls == 1 and first.rewards.shape == (2, 3)
    again, fresh = runner(BATCH)
    assert not fresh and again is first and reward.calls == 1
    other, fresh = runner({"messages": BATCH["messages"][:1]})
    assert fresh and other is not first  # another prompt batch is never served from the cache
    runner(BATCH)
    runner.step()
    assert not runner(BATCH)[1]
    runner.step()
    assert runner(BATCH)[1]  # two optimizer steps: the interval is reached
    assert not runner(BATCH)[1]  # ... and the counter started again
    runner.clear_cache()
    assert runner(BATCH)[1]


def test_online_grpo_runs_rollouts_and_syncs_the_old_policy_on_refresh(tok):
    model = _model()
    s = _grpo(model)
    runner, _ = _runner(tok, model, interval=2)
    s.set_rollout_runner(runner)
    with torch.no_grad():
        for p in s.old_model.parameters():
            p.mul_(0.5)  # make the old policy visibly different
    out = s(BATCH)
    assert torch.isfinite(out["loss"])
    assert all(torch.equal(a, b) for a, b in zip(model.state_dict().values(), s.old_model.state_dict().values()))  # synced on refresh
    with torch.no_grad():
        for p in model.parameters():
            p.add_(0.01)
    s(BATCH)  # cached rollout: no refresh, the old policy stays where it was
    assert any(not torch.equal(a, b) for a, b in zip(model.state_dict().values(), s.old_model.state_dict().values()))
    s.on_optimizer_step()
    s.on_optimizer_step()
    s(BATCH)  # interval reached: new rollout, old policy synced again
    assert all(torch.equal(a, b) for a, b in zip(model.state_dict().values(), s.old_model.state_dict().values()))


def test_online_dpo_picks_best_and_worst_of_each_group(tok):
    from astrai_b200.trainer.rollout import RolloutResult

    s = _dpo()
    responses = torch.arange(2 * 3 * 4).reshape(2, 3, 4) + 5
    mask = torch.ones(2, 3, 4, dtype=torch.bool)
    mask[0, 2, 2:] = False
    result = RolloutResult(prompts=torch.ones(2, 2, dtype=torch.long), prompt_mask=torch.ones(2, 2, dtype=torch.bool), responses=responses,
                           response_mask=mask, logprobs_old=torch.zeros(2, 3, 4), rewards=torch.tensor([[0.1, 0.9, 0.5], [2.0, -1.0, 0.0]]))
    batch = s.prepare_from_rollout(result)
    assert torch.equal(batch["chosen"], responses[[0, 1], [1, 0]]) and torch.equal(batch["rejected"], responses[[0, 1], [0, 1]])
    assert batch["chosen_mask"].shape == (2, 4) and batch["rejected_mask"][0].tolist() == [1.0, 1.0, 1.0, 1.0]
    model = _model()
    online = _dpo(model)
    runner, _ = _runner(tok, model)
    online.set_rollout_runner(runner)
    out = online(BATCH)
    assert torch.isfinite(out["loss"]) and out["loss"].requires_grad


def test_offline_call_without_runner_uses_the_batch_itself():
    s = _grpo()
    batch = _grpo_batch()
    assert float(s(batch)["loss"]) == pytest.approx(float(s.compute_loss_output(batch)["loss"]), abs=1e-7)
    s.on_optimizer_step()  # no runner: a no-op


# ------------------------------------------------------------------------------------------------------ loss output
def test_moe_aux_loss_is_weighted_into_the_total_and_reported():
    from astrai_b200.trainer import StrategyFactory

    model = _model(ffn_type="moe", n_routed_experts=4, n_shared_experts=1, n_activated_experts=2, moe_intermediate_size=32).train()
    ids = torch.randint(3, 500, (2, 17))
    batch = {"input_ids": ids[:, :-1], "target_ids": ids[:, 1:]}
    out = StrategyFactory.create("seq", model=model, device="cpu", moe_aux_loss_coef=0.5)(batch)
    m = out["metrics"].resolved()
    assert m["moe_aux_loss_weighted"] == pytest.approx(0.5 * m["moe_aux_loss"], rel=1e-5)
    zero = StrategyFactory.create("seq", model=model, device="cpu", moe_aux_loss_coef=0.0)(batch)
    z = zero["metrics"].resolved()
    assert z["moe_aux_loss_weighted"] == 0.0 and z["moe_aux_loss"] > 0
    assert float(out["loss"]) == pytest.approx(float(zero["loss"]) + m["moe_aux_loss_weighted"], rel=1e-5)
    dense = StrategyFactory.create("seq", model=_model(), device="cpu")(batch)
    assert "moe_aux_loss" not in dense["metrics"]


def test_plain_tensor_losses_are_wrapped():
    from astrai_b200.trainer.strategy import BaseStrategy

    class Legacy(BaseStrategy):
        def compute_loss(self, batch):
            return batch["x"].sum()

    out = Legacy(torch.nn.Identity(), "cpu")({"x": torch.tensor([1.0, 2.0], requires_grad=True)})
    assert float(out["loss"]) == 3.0 and out["metrics"].resolved() == {"loss": 3.0}
