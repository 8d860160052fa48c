"""Interrupted runs: stop signals (both kinds, and one that arrives before the trainer exists), checkpoints written on
the way out, and resumed runs that continue exactly where the interrupted one stopped."""

import os
import signal
import subprocess
import sys
import textwrap

import pytest
import torch

from helpers import RandomTokens
from test_trainer import _train_config

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


@pytest.fixture
def handlers():
    from astrai_b200 import signal_handler as sh

    yield sh
    sh.unregister_signal_handlers()
    signal.signal(signal.SIGTERM, signal.SIG_DFL)
    signal.signal(signal.SIGINT, signal.default_int_handler)


class _Ctx:
    def __init__(self):
        self.stops = 0

    def request_stop(self):
        self.stops += 1


def test_context_stop_flag():
    from astrai_b200.trainer.train_context import TrainContext

    ctx = TrainContext()
    assert not ctx.stop_requested
    ctx.request_stop()
    assert ctx.stop_requested


@pytest.mark.parametrize("sig", [signal.SIGTERM, signal.SIGINT])
def test_either_signal_requests_a_stop(handlers, sig):
    ctx = _Ctx()
    handlers.register_signal_handlers(ctx)
    assert ctx.stops == 0
    os.kill(os.getpid(), sig)
    assert ctx.stops == 1


def test_signal_before_the_context_exists_is_replayed(handlers):
    handlers.install_early_signal_handlers()
    os.kill(os.getpid(), signal.SIGTERM)  # nothing to stop yet: remembered
    ctx = _Ctx()
    handlers.register_signal_handlers(ctx)
    assert ctx.stops == 1


def test_unregister_forgets_the_context_and_the_pending_signal(handlers):
    first = _Ctx()
    handlers.register_signal_handlers(first)
    os.kill(os.getpid(), signal.SIGTERM)
    handlers.unregister_signal_handlers()
    second = _Ctx()
    handlers.register_signal_handlers(second)
    assert first.stops == 1 and second.stops == 0
    os.kill(os.getpid(), signal.SIGINT)
    assert first.stops == 1 and second.stops == 1


@pytest.mark.parametrize("sig", ["SIGTERM", "SIGINT"])
def test_signal_in_mid_run_leaves_a_resumable_checkpoint(tmp_path, sig):
    script = textwrap.dedent(f"""
        import os, signal, sys
        sys.path.insert(0, {ROOT!r}); sys.path.insert(0, {HERE!r})
        from test_trainer import _train_config
        from helpers import RandomTokens
        from astrai_b200.trainer import Trainer
        class Interrupt:
            seen = 0
            def on_batch_end(self, ctx):
                Interrupt.seen += 1
                if Interrupt.seen == 5:
                    os.kill(os.getpid(), signal.{sig})
        Trainer(_train_config({str(tmp_path)!r}, dataset=RandomTokens(400, 12), ckpt_interval=10**6, n_epoch=50),
                callbacks=[Interrupt()]).train()
    """)
    proc = subprocess.run([sys.executable, "-c", script], capture_output=True, text=True, timeout=180)
    assert proc.returncode == 0, proc.stderr[-2000:]
    from astrai_b200.serialization import Checkpoint, latest_complete

    ck_dir = latest_complete(tmp_path)
    assert ck_dir is not None, proc.stderr[-2000:]
    ck = Checkpoint.load(ck_dir)
    # stopped between steps, long before the 50 epochs: whole micro-batches of 2 samples, a handful of them
    assert 0 < ck.consumed_samples <= 16 and ck.consumed_samples % 2 == 0
    assert "optimizer" in ck.extra and "scheduler" in ck.extra


class _StopAfter:
    def __init__(self, steps):
        self.steps = steps

    def on_batch_end(self, ctx):
        if ctx.consumed_samples >= self.steps * 4:  # 2 samples per micro-batch, 2 micro-batches per optimizer step
            ctx.request_stop()


def _final_weights(directory):
    from astrai_b200.serialization import Checkpoint, latest_complete

    ck = Checkpoint.load(latest_complete(directory))
    return ck, {k: v.clone() for k, v in ck.state_dict.items()}


@pytest.mark.parametrize("stop_at", [3, 10, 17])
def test_resumed_run_ends_where_an_uninterrupted_one_does(tmp_path, stop_at):
    """Two epochs of 10 optimizer steps each; stopping inside the first or the second epoch and resuming from the
    checkpoint written on the way out gives the weights, step count and learning rate of a run that never stopped."""
    from astrai_b200.trainer import Trainer

    whole, parts = tmp_path / "whole", tmp_path / "parts"
    kw = dict(n_epoch=2, ckpt_interval=10**6, random_seed=7)
    Trainer(_train_config(whole, dataset=RandomTokens(40, 12), **kw)).train()
    ck_whole, w_whole = _final_weights(whole)

    trainer = Trainer(_train_config(parts, dataset=RandomTokens(40, 12), **kw))
    trainer.callbacks.append(_StopAfter(stop_at))
    trainer.train()
    ck_part, _ = _final_weights(parts)
    assert ck_part.consumed_samples == stop_at * 4
    Trainer(_train_config(parts, dataset=RandomTokens(40, 12), **kw)).train(param_path=_latest(parts), resume=True)
    ck_res, w_res = _final_weights(parts)
    assert ck_res.consumed_samples == ck_whole.consumed_samples == 80
    for name, ref in w_whole.items():
        assert torch.equal(w_res[name], ref), name
    assert ck_res.extra["scheduler"]["last_epoch"] == ck_whole.extra["scheduler"]["last_epoch"]


def _latest(directory):
    from astrai_b200.serialization import latest_complete

    return str(latest_complete(directory))


def test_resume_rounds_down_to_a_whole_optimizer_step(tmp_path):
    """A checkpoint written in the middle of an accumulation window resumes at the window's start: the half-built
    gradient is not in the checkpoint, so its samples are taken again."""
    from astrai_b200.serialization import Checkpoint, latest_complete
    from astrai_b200.trainer import Trainer
    from astrai_b200.trainer.train_context import TrainContextBuilder

    with pytest.raises(RuntimeError, match="injected"):
        Trainer(_train_config(tmp_path, dataset=RandomTokens(40, 12, fail_after=14), ckpt_interval=10**6)).train()
    ck_dir = latest_complete(tmp_path)
    assert Checkpoint.load(ck_dir).consumed_samples == 14  # 7 micro-batches of 2: 3 optimizer steps and a half
    ctx = TrainContextBuilder(_train_config(tmp_path)).with_param_path(str(ck_dir), resume=True).build()
    assert ctx.consumed_samples == 12 and ctx.optimizer_step == 3


def test_param_path_without_resume_loads_weights_only(tmp_path):
    from astrai_b200.serialization import latest_complete
    from astrai_b200.trainer import Trainer
    from astrai_b200.trainer.train_context import TrainContextBuilder

    Trainer(_train_config(tmp_path / "a", ckpt_interval=10**6)).train()
    ck_dir = latest_complete(tmp_path / "a")
    ctx = TrainContextBuilder(_train_config(tmp_path / "b")).with_param_path(str(ck_dir), resume=False).build()
    assert ctx.consumed_samples == 0 and ctx.optimizer_step == 0 and ctx.epoch == 0
    from astrai_b200.serialization import Checkpoint

    saved = Checkpoint.load(ck_dir).state_dict
    for name, value in ctx.model.state_dict().items():
        assert torch.equal(value, saved[name]), name
