"""Trainer callbacks and the metric log: requested metrics only, strategy-supplied metrics, validation rows, flush rules,
gradient statistics, the progress bar, activation checkpointing, batch-size / accumulation arithmetic (behaviours the
reference checks in ``tests/trainer/test_callbacks.py``, ``test_loss_output.py``, ``test_metric_util.py``,
``test_early_stopping.py`` and ``test_trainer.py``)."""

import io
import json
import os

import pytest
import torch

from helpers import RandomTokens, tiny_config


def _model():
    from astrai_b200.models import AutoRegressiveLM

    torch.manual_seed(0)
    return AutoRegressiveLM(tiny_config(tie_word_embeddings=True))


def _moe_model():
    from astrai_b200.models import AutoRegressiveLM

    torch.manual_seed(0)
    return AutoRegressiveLM(tiny_config(ffn_type="moe", n_routed_experts=4, n_shared_experts=1, n_activated_experts=2))


def _opt(model):
    return torch.optim.AdamW(model.parameters(), lr=1e-2)


def _config(tmp, **over):
    from astrai_b200.config import TrainConfig

    base = dict(model_fn=_model, strategy="seq", dataset=RandomTokens(24, 12), optimizer_fn=_opt, batch_per_device=2,
                grad_accum_steps=2, ckpt_dir=str(tmp), ckpt_interval=100, device_type="cpu", backend="gloo", master_port=None)
    base.update(over)
    return TrainConfig(**base)


def _rows(tmp):
    last = sorted((p for p in os.listdir(tmp) if p.startswith("epoch_")), key=lambda n: int(n.split("_")[-1]))[-1]
    return [json.loads(line) for line in open(os.path.join(tmp, last, "metric.jsonl"))]


# --------------------------------------------------------------------------------------------------------- metric log
def test_metric_log_holds_the_requested_metrics_per_optimizer_step(tmp_path):
    from astrai_b200.trainer import Trainer

    Trainer(_config(tmp_path, metrics=["loss", "lr"])).train()
    rows = _rows(tmp_path)
    steps = [r for r in rows if r["type"] == "step"]
    assert len(steps) == 6 and [r["step"] for r in steps] == list(range(1, 7))      # 24 samples / (2 x 2) per step
    assert all({"loss", "lr", "epoch", "consumed_samples", "timestamp"} <= set(r) for r in steps)
    assert all("grad_norm" not in r and "grad_snr" not in r for r in steps)           # not asked for, not computed
    assert [r["consumed_samples"] for r in steps] == [4 * i for i in range(1, 7)]
    assert [r["type"] for r in rows if r["type"] != "step"] == ["epoch"]


def test_metric_log_adds_gradient_statistics_on_request(tmp_path):
    from astrai_b200.trainer import Trainer

    Trainer(_config(tmp_path, metrics=["loss", "grad_norm", "grad_snr"], max_grad_norm=0.5)).train()
    steps = [r for r in _rows(tmp_path) if r["type"] == "step"]
    assert all(r["grad_norm"] > 0 and isinstance(r["grad_snr"], float) for r in steps)


def test_metric_log_carries_what_the_strategy_reports(tmp_path):
    from astrai_b200.trainer import Trainer

    Trainer(_config(tmp_path, model_fn=_moe_model, metrics=["loss", "moe_aux_loss", "router_entropy", "dead_expert_fraction"])).train()
    step = [r for r in _rows(tmp_path) if r["type"] == "step"][0]
    assert {"moe_aux_loss", "moe_aux_loss_weighted", "router_entropy", "dead_expert_fraction"} <= set(step)
    assert 0 <= step["dead_expert_fraction"] <= 1 and step["router_entropy"] > 0
    dense = tmp_path / "dense"
    Trainer(_config(dense, metrics=["loss", "moe_aux_loss", "router_entropy"])).train()
    assert all("router_entropy" not in r for r in _rows(dense) if r["type"] == "step")  # nothing to report for a dense model


def test_validation_runs_every_val_step_and_is_logged(tmp_path):
    from astrai_b200.trainer import Trainer

    t = Trainer(_config(tmp_path, val_dataset=RandomTokens(8, 12, seed=5), val_step=2, metrics=["loss", "val_loss"]))
    t.train()
    rows = _rows(tmp_path)
    val = [r for r in rows if r["type"] == "validation"]
    assert [r["step"] for r in val] == [1, 3, 5] and all(r["val_loss"] > 0 for r in val)
    # a validation pass leaves the model in training mode and does not touch the step count
    assert [r["step"] for r in rows if r["type"] == "step"] == list(range(1, 7))


def test_val_split_takes_samples_away_from_training(tmp_path):
    from astrai_b200.trainer import Trainer

    Trainer(_config(tmp_path, dataset=RandomTokens(40, 12), val_split=0.2, val_step=100)).train()
    steps = [r for r in _rows(tmp_path) if r["type"] == "step"]
    assert len(steps) == 8 and steps[-1]["consumed_samples"] == 32  # 32 of 40 samples train; 8 are held out


def test_metric_log_is_flushed_at_the_save_interval_and_at_the_end(tmp_path):
    from astrai_b200.trainer import Trainer

    Trainer(_config(tmp_path, ckpt_interval=2)).train()
    with_log = sorted(int(d.split("_")[-1]) for d in os.listdir(tmp_path) if os.path.exists(tmp_path / d / "metric.jsonl"))
    assert with_log == [2, 4, 6]
    assert len([1 for line in open(tmp_path / "epoch_0_step_4" / "metric.jsonl") if '"step"' in line]) >= 4  # cumulative


def test_metric_log_survives_a_crash(tmp_path):
    from astrai_b200.trainer import Trainer

    with pytest.raises(RuntimeError, match="injected"):
        Trainer(_config(tmp_path, dataset=RandomTokens(24, 12, fail_after=10))).train()
    steps = [r for r in _rows(tmp_path) if r["type"] == "step"]
    assert len(steps) == 2  # the two completed optimizer steps were written by the error hook


# ----------------------------------------------------------------------------------------------------- grad statistics
def test_grad_norm_totals_and_per_parameter_values():
    from astrai_b200.trainer.metric_util import grad_norm

    m = torch.nn.Sequential(torch.nn.Linear(3, 2), torch.nn.Linear(2, 1))
    assert grad_norm(m) == 0.0
    m(torch.ones(4, 3)).sum().backward()
    per = grad_norm(m, per_param=True)
    want = sum(p.grad.pow(2).sum() for p in m.parameters()).sqrt().item()
    assert per["total"] == pytest.approx(want) == pytest.approx(grad_norm(m))
    assert set(per) == {"0.weight", "0.bias", "1.weight", "1.bias", "total"} and per["1.bias"] == pytest.approx(4.0)


def test_grad_snr_is_high_for_steady_gradients_and_low_for_noise():
    from astrai_b200.trainer.metric_util import GradSNRTracker

    lin = torch.nn.Linear(64, 64)
    steady, noisy = GradSNRTracker(beta=0.9), GradSNRTracker(beta=0.9)
    assert steady.snr == 0.0
    g = torch.Generator().manual_seed(0)
    signal = torch.randn(64, 64, generator=g)
    for _ in range(60):
        lin.weight.grad, lin.bias.grad = signal + 0.01 * torch.randn(64, 64, generator=g), torch.zeros(64)
        steady.update(lin)
        lin.weight.grad = torch.randn(64, 64, generator=g)
        noisy.update(lin)
    assert steady.snr > 10.0 and noisy.snr < 0.0 and steady.snr > noisy.snr + 15.0  # dB


# ------------------------------------------------------------------------------------------------------- progress bar
def test_progress_bar_reports_step_loss_lr_and_norm(tmp_path):
    from astrai_b200.trainer import CallbackFactory, Trainer

    buf = io.StringIO()
    t = Trainer(_config(tmp_path, max_grad_norm=1.0))
    t.callbacks = [cb for cb in t.callbacks if type(cb).__name__ != "ProgressBarCallback"]
    t.callbacks.append(CallbackFactory.create("progress_bar", 1, file=buf))
    t.train()
    text = buf.getvalue()
    assert "Epoch 1/1" in text and "loss=" in text and "lr=" in text and "grad_norm=" in text and "step=6" in text


# --------------------------------------------------------------------------------------------- activation checkpointing
def test_activation_checkpointing_wraps_and_unwraps_only_the_listed_modules():
    from astrai_b200.models.decoder import DecoderBlock
    from astrai_b200.trainer import CallbackFactory

    model = _model()
    ctx = type("Ctx", (), {"model": model})()
    cb = CallbackFactory.create("gradient_checkpointing", modules=[DecoderBlock])
    cb.on_train_begin(ctx)
    wrapped = [m for m in model.modules() if hasattr(m, "_plain_forward")]
    assert len(wrapped) == len(model.layers) and all(isinstance(m, DecoderBlock) for m in wrapped)
    cb.on_train_begin(ctx)  # a second call must not wrap the wrapper
    assert all(not hasattr(m._plain_forward, "__wrapped_twice__") for m in wrapped)
    ids = torch.randint(0, 1000, (2, 9))
    out = model(ids)["logits"]
    out.sum().backward()
    assert all(p.grad is not None for p in model.layers[0].parameters())
    cb.on_train_end(ctx)
    assert not any(hasattr(m, "_plain_forward") for m in model.modules())
    noop = CallbackFactory.create("gradient_checkpointing", modules=None)
    noop.on_train_begin(ctx)
    assert not any(hasattr(m, "_plain_forward") for m in model.modules())


def test_activation_checkpointing_keeps_outputs_and_gradients():
    from astrai_b200.models.decoder import DecoderBlock
    from astrai_b200.trainer import CallbackFactory

    ids = torch.randint(0, 1000, (2, 9))
    plain, ckpt = _model(), _model()
    ctx = type("Ctx", (), {"model": ckpt})()
    CallbackFactory.create("gradient_checkpointing", modules=[DecoderBlock]).on_train_begin(ctx)
    a, b = plain(ids)["logits"], ckpt(ids)["logits"]
    assert torch.allclose(a, b, atol=1e-6)
    a.pow(2).mean().backward()
    b.pow(2).mean().backward()
    for (n, p), q in zip(plain.named_parameters(), ckpt.parameters()):
        assert torch.allclose(p.grad, q.grad, atol=1e-6), n


# ------------------------------------------------------------------------------------------- batch / accumulation sizes
@pytest.mark.parametrize("bpd,accum,samples,steps", [(1, 1, 10, 10), (2, 1, 10, 5), (4, 2, 24, 3), (3, 2, 20, 3), (8, 4, 24, 0)])
def test_step_count_follows_batch_size_and_accumulation(tmp_path, bpd, accum, samples, steps):
    from astrai_b200.trainer import Trainer

    t = Trainer(_config(tmp_path, dataset=RandomTokens(samples, 12), batch_per_device=bpd, grad_accum_steps=accum))
    t.train()
    if steps == 0:  # fewer micro-batches than one accumulation window: no optimizer step was taken
        logs = [d for d in os.listdir(tmp_path) if os.path.exists(tmp_path / d / "metric.jsonl")]
        assert not logs or not [r for r in _rows(tmp_path) if r["type"] == "step"]
        return
    assert len([r for r in _rows(tmp_path) if r["type"] == "step"]) == steps


def test_two_epochs_continue_the_step_count_and_reshuffle(tmp_path):
    from astrai_b200.trainer import Trainer

    Trainer(_config(tmp_path, n_epoch=2)).train()
    rows = _rows(tmp_path)
    steps = [r for r in rows if r["type"] == "step"]
    assert [r["step"] for r in steps] == list(range(1, 13)) and [r["epoch"] for r in steps] == [0] * 6 + [1] * 6
    assert [r["epoch"] for r in rows if r["type"] == "epoch"] == [0, 1]
    assert steps[-1]["consumed_samples"] == 48


def test_loss_denominator_turns_slice_means_into_the_mean_over_all_trained_tokens():
    """Two ranks hold halves of a batch with 1 and 5 trained tokens: with the shared denominator the average of their
    losses (and of their gradients) is the whole batch's mean; without it, it is not."""
    from astrai_b200 import ops

    torch.manual_seed(0)
    logits = torch.randn(12, 9, requires_grad=True)
    targets = torch.randint(0, 9, (12,))
    keep = torch.tensor([1, 0, 0, 0, 0, 0, 1, 1, 0, 1, 1, 1], dtype=torch.bool)
    targets = targets.masked_fill(~keep, -100)
    whole = ops.cross_entropy(logits, targets)
    whole.backward()
    ref_grad, logits.grad = logits.grad.clone(), None

    halves = []
    with ops.loss_denominator(keep.sum().float() / 2):
        for r in range(2):
            halves.append(ops.cross_entropy(logits[r * 6:(r + 1) * 6], targets[r * 6:(r + 1) * 6]))
    (sum(halves) / 2).backward()
    assert float((sum(halves) / 2).detach()) == pytest.approx(float(whole.detach()), rel=1e-6)
    assert torch.allclose(logits.grad, ref_grad, atol=1e-7)

    plain = [ops.cross_entropy(logits[r * 6:(r + 1) * 6], targets[r * 6:(r + 1) * 6]) for r in range(2)]
    assert abs(float((sum(plain) / 2).detach()) - float(whole.detach())) > 1e-3  # the slices' own counts weight the tokens unevenly
    with ops.loss_denominator(None):
        assert float(ops.cross_entropy(logits, targets).detach()) == pytest.approx(float(whole.detach()))
    # the context ends with the block
    assert float(ops.cross_entropy(logits[:6], targets[:6]).detach()) == pytest.approx(float(plain[0].detach()))
