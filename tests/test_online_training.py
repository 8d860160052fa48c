"""Online reinforcement learning through the real Trainer: prompts from a dataset of instructions, responses sampled by
the policy through the serving scheduler, scored by a rule, trained on with GRPO / DPO (CPU, one process)."""

import json
import os

import pytest
import torch

from helpers import TINY, build_tokenizer_dir


class Instructions(torch.utils.data.Dataset):
    ROWS = [{"instruction": "Hello", "input": ""}, {"instruction": "Tell me a story", "input": "about dragons"},
            {"instruction": "Summarize", "input": "the article"}, {"instruction": "Translate", "input": "to French: hi"}]

    def __len__(self):
        return len(self.ROWS)

    def __getitem__(self, i):
        return dict(self.ROWS[i])


def collate(batch):
    return {"instruction": [b["instruction"] for b in batch], "input": [b.get("input", "") for b in batch]}


class LongerIsBetter:
    """Reward = number of characters of the response (a rule, not a model); remembers what it scored."""

    seen = []

    def score(self, prompts, responses):
        LongerIsBetter.seen.append((list(prompts), [list(r) for r in responses]))
        return torch.tensor([[float(len(text)) for text in group] for group in responses])


def _model():
    from astrai_b200.config import AutoRegressiveLMConfig
    from astrai_b200.models import AutoRegressiveLM

    torch.manual_seed(5)
    return AutoRegressiveLM(AutoRegressiveLMConfig(**{**TINY, "vocab_size": 512, "max_position_embeddings": 128}))


def _adamw(model):
    return torch.optim.AdamW(model.parameters(), lr=1e-3)


@pytest.mark.parametrize("strategy,kwargs", [("online_grpo", {"clip_eps": 0.2, "kl_coef": 0.01, "group_size": 2}),
                                             ("online_dpo", {"beta": 0.1, "group_size": 2})])
def test_online_rollout_training_end_to_end(tmp_path, strategy, kwargs):
    from astrai_b200.config import TrainConfig
    from astrai_b200.serialization import Checkpoint, latest_complete
    from astrai_b200.trainer import Trainer

    params = build_tokenizer_dir(str(tmp_path / "params"))
    LongerIsBetter.seen = []
    cfg = TrainConfig(strategy=strategy, model_fn=_model, dataset=Instructions(), optimizer_fn=_adamw, ckpt_dir=str(tmp_path / "ck"),
                      n_epoch=1, batch_per_device=2, grad_accum_steps=1, ckpt_interval=100, random_seed=42, device_type="cpu", backend="gloo",
                      nprocs=1, parallel_mode="none", strategy_kwargs=kwargs, rollout_interval=1, rollout_temperature=1.0, rollout_top_k=0,
                      rollout_top_p=1.0, rollout_max_tokens=4, reward_model_fn=LongerIsBetter, collate_fn=collate, metrics=["loss"])
    Trainer(cfg).train(param_path=params)

    ck = Checkpoint.load(latest_complete(tmp_path / "ck"))
    assert ck.consumed_samples == 4
    start = _model().state_dict()
    assert any(not torch.equal(ck.state_dict[k], start[k]) for k in start)  # the policy learned something
    # two batches of two prompts, two sampled responses each, rendered through the chat template
    assert len(LongerIsBetter.seen) == 2
    for prompts, responses in LongerIsBetter.seen:
        assert len(prompts) == 2 and [len(r) for r in responses] == [2, 2]
        assert all("<|im_start|>" in p and p.endswith("<|im_start|>assistant\n") for p in prompts)
        assert all(isinstance(text, str) for group in responses for text in group)
    rows = [json.loads(line) for line in open(os.path.join(latest_complete(tmp_path / "ck"), "metric.jsonl"))]
    steps = [r for r in rows if r["type"] == "step"]
    assert len(steps) == 2 and all(torch.isfinite(torch.tensor(r["loss"])) for r in steps)


def test_offline_strategy_name_with_online_data_is_refused(tmp_path):
    from astrai_b200.config import TrainConfig

    with pytest.raises(ValueError):
        TrainConfig(strategy="online_sft", model_fn=_model, dataset=Instructions(), optimizer_fn=_adamw)


def test_online_rollouts_are_refused_where_the_training_model_has_no_serving_forward(tmp_path):
    from astrai_b200.config import TrainConfig
    from astrai_b200.trainer.train_context import TrainContextBuilder

    class Strategy:
        def supports_online(self):
            return True

    class Ctx:
        strategy = Strategy()

    for mode in ("tp", "cp", "pp"):
        cfg = TrainConfig(strategy="online_grpo", model_fn=_model, dataset=Instructions(), optimizer_fn=_adamw, parallel_mode=mode, reward_model_fn=LongerIsBetter,
                          nprocs=2, device_type="cpu", backend="gloo", ckpt_dir=str(tmp_path))
        with pytest.raises(ValueError, match="online rollouts sample from the training model"):
            TrainContextBuilder(cfg)._rollout(Ctx(), {})
