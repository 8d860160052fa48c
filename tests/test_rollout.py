"""Rollout generator / runner with a scripted scheduler and tokenizer (no model): packing, caching, refresh."""

import pytest
import torch

from astrai_b200.trainer.rollout import BaseRewardModel, RolloutGenerator, RolloutResult, RolloutRunner, messages_from_fields


class _Tok:
    stop_ids = [1]

    def apply_chat_template(self, conv, tokenize=False, add_generation_prompt=True):
        if conv and isinstance(conv[0], list):
            raise TypeError("single conversations only")
        text = "|".join(f"{m['role']}:{m['content']}" for m in conv) + "|assistant:"
        return [ord(c) % 50 + 2 for c in text] if tokenize else text

    def decode(self, ids, skip_special_tokens=True):
        return " ".join(str(i) for i in ids)


class _Sched:
    device = torch.device("cpu")

    def __init__(self):
        self.calls = 0
        self._executor = type("E", (), {"model": torch.nn.Linear(2, 2)})()

    def run_batch(self, prompts, *, max_tokens, return_logprobs, **sampling):
        self.calls += 1
        assert return_logprobs and not self._executor.model.training  # generation runs in eval mode
        out = []
        for i, p in enumerate(prompts):
            n = (i % 3) + (1 if i % 2 == 0 else 0)  # some empty generations
            out.append(([10 + i + k for k in range(n)], [-0.5 * (k + 1) for k in range(n)]))
        return out


class _LenReward(BaseRewardModel):
    def score(self, prompts, responses):
        return torch.tensor([[float(len(r.split())) if r else 0.0 for r in row] for row in responses])


def test_messages_from_fields_skips_empty():
    assert messages_from_fields("be brief", "", "") == [{"role": "system", "content": "be brief"}]
    assert [m["role"] for m in messages_from_fields("a", "b", "c")] == ["system", "user", "assistant"]


def test_generator_packs_left_padded_prompts_and_right_padded_responses():
    sched = _Sched()
    sched._executor.model.train()
    gen = RolloutGenerator(sched, _Tok(), max_tokens=8, group_size=2, temperature=0.7)
    raw = gen.generate({"instruction": ["short", "a much longer instruction"], "input": ["x", ""]})
    assert sched._executor.model.training  # restored
    b, g, r = raw.responses.shape
    assert (b, g) == (2, 2) and raw.prompts.shape[0] == 2
    assert raw.prompt_mask[1].all() and not raw.prompt_mask[0, 0]  # the shorter prompt is padded on the left
    assert raw.prompt_mask[0].sum() == len(_Tok().apply_chat_template(messages_from_fields("short", "x"), tokenize=True))
    lens = raw.response_mask.sum(-1)
    assert lens.tolist() == [[1, 1], [3, 0]]
    assert raw.responses[1, 0, :3].tolist() == [12, 13, 14] and raw.logprobs_old[1, 0, :3].tolist() == [-0.5, -1.0, -1.5]
    assert (raw.responses[~raw.response_mask] == 0).all()
    assert raw.response_texts[1][1] == ""


def test_runner_caches_per_batch_and_refreshes_on_interval():
    sched = _Sched()
    runner = RolloutRunner(RolloutGenerator(sched, _Tok(), group_size=2), _LenReward(), rollout_interval=2)
    batch = {"messages": [[{"role": "user", "content": "hi"}]]}
    first, fresh = runner(batch)
    assert fresh and isinstance(first, RolloutResult) and first.rewards.shape == (1, 2)
    again, fresh = runner(batch)
    assert not fresh and again is first and sched.calls == 1
    runner.step()
    assert not runner(batch)[1]
    runner.step()
    assert runner(batch)[1] and sched.calls == 2  # interval reached
    assert runner({"messages": [[{"role": "user", "content": "other"}]]})[1]  # a different batch is never served stale
    with pytest.raises(ValueError):
        RolloutGenerator(sched, _Tok()).generate({"text": ["x"]})
