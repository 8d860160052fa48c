"""Factory, configs, schedulers, sampler: behaviour contracts of the pure-Python core."""

import json
import math

import pytest
import torch

from astrai_b200.factory import BaseFactory


class _Base:
    pass


class _F(BaseFactory[_Base]):
    pass


def test_factory_register_create_filters_kwargs():
    @_F.register("a")
    class A(_Base):
        def __init__(self, x, y=2):
            self.x, self.y = x, y

    obj = _F.create("a", 1, y=5, unrelated=7)
    assert (obj.x, obj.y) == (1, 5)
    assert _F.is_registered("a") and "a" in _F.list_registered()
    with pytest.raises(ValueError):
        _F.register("a")(A)
    with pytest.raises(TypeError):
        _F.register("b")(int)
    with pytest.raises(ValueError):
        _F.create("missing")


def test_factory_passes_var_kwargs_through():
    @_F.register("kw")
    class K(_Base):
        def __init__(self, **kw):
            self.kw = kw

    assert _F.create("kw", p=1, q=2).kw == {"p": 1, "q": 2}


def test_model_config_roundtrip(tmp_path):
    from astrai_b200.config import AutoRegressiveLMConfig, ConfigFactory, EncoderConfig

    cfg = AutoRegressiveLMConfig(vocab_size=10, hidden_size=8, num_attention_heads=2, ffn_type="moe", n_routed_experts=4)
    p = tmp_path / "config.json"
    cfg.to_file(p)
    raw = json.loads(p.read_text())
    assert "q_lora_rank" not in raw and raw["norm_topk_prob"] is True and raw["moe_aux_loss_coef"] == 0.01
    assert ConfigFactory.load(raw) == cfg
    assert isinstance(ConfigFactory.load({"model_type": "embedding", "pooling_type": "cls"}), EncoderConfig)
    with pytest.raises(Exception):
        AutoRegressiveLMConfig(attn_type="bogus")
    with pytest.raises(Exception):
        AutoRegressiveLMConfig(decoder_sparse_step=0)


def test_train_config_validation_and_to_dict():
    from astrai_b200.config import TrainConfig

    base = dict(model_fn=lambda: None, strategy="seq", dataset=[1], optimizer_fn=lambda m: None, scheduler_fn=lambda o: None)
    cfg = TrainConfig(**base)
    d = cfg.to_dict()
    assert "model_fn" not in d and d["strategy"] == "seq" and d["batch_per_device"] == 4
    for bad in (dict(strategy="nope"), dict(parallel_mode="x"), dict(backend="mpi"), dict(grad_accum_steps=0),
                dict(val_split=1.5), dict(max_grad_norm=-1.0), dict(strategy="online_grpo")):
        with pytest.raises(Exception):
            TrainConfig(**{**base, **bad})


@pytest.mark.parametrize("name,kw", [("cosine", dict(warmup_steps=4, lr_decay_steps=20)),
                                     ("sgdr", dict(warmup_steps=2, cycle_length=5, t_mult=2)),
                                     ("wsd", dict(warmup_steps=3, stable_steps=5, decay_steps=10))])
def test_schedulers_formula_and_state(name, kw):
    from astrai_b200.trainer import SchedulerFactory

    p = torch.nn.Parameter(torch.zeros(1))
    opt = torch.optim.SGD([p], lr=1.0)
    sch = SchedulerFactory.create(name, opt, **kw)
    seen = []
    for _ in range(30):
        seen.append(opt.param_groups[0]["lr"])
        opt.step()
        sch.step()
    assert seen[0] == pytest.approx(0.01)  # warm-up floor = min_rate
    assert max(seen) <= 1.0 + 1e-9 and min(seen) >= 0.01 - 1e-9
    if name == "cosine":
        step = 14
        expect = max(0.01, 0.5 * (1 + math.cos(math.pi * (step - 4) / 20)))
        assert seen[step] == pytest.approx(expect)
        assert seen[-1] == pytest.approx(0.01)
    if name == "wsd":
        assert seen[5] == 1.0 and seen[3 + 5 + 5] == pytest.approx(0.99 * 0.25 + 0.01)
    if name == "sgdr":
        assert seen[2] == pytest.approx(1.0) and seen[7] == pytest.approx(1.0)  # restarts
    state = sch.state_dict()
    assert "warmup_steps" in state
    opt2 = torch.optim.SGD([p], lr=1.0)
    sch2 = SchedulerFactory.create(name, opt2, **{k: 1 for k in kw})
    sch2.load_state_dict(state)
    assert sch2.last_epoch == sch.last_epoch and sch2.warmup_steps == kw["warmup_steps"]


def test_rd_sampler_resume_and_sharding():
    from astrai_b200.data import RDSampler

    data = list(range(10))
    full = list(RDSampler(data, seed=1))
    assert sorted(full) == data
    resumed = list(RDSampler(data, seed=1, start_iter=4))
    assert resumed == full[4:]
    s = RDSampler(data, seed=1)
    first = list(s)
    second = list(s)
    assert first != second and sorted(second) == data  # reshuffled next epoch
    assert list(RDSampler(data, shuffle=False)) == data


def test_signal_handler_requests_stop():
    import os
    import signal

    from astrai_b200 import signal_handler as sh

    class Ctx:
        stopped = False

        def request_stop(self):
            self.stopped = True

    ctx = Ctx()
    sh.register_signal_handlers(ctx)
    try:
        os.kill(os.getpid(), signal.SIGTERM)
        assert ctx.stopped
    finally:
        sh.unregister_signal_handlers()
        signal.signal(signal.SIGTERM, signal.SIG_DFL)
        signal.signal(signal.SIGINT, signal.default_int_handler)


def test_attention_backend_selection(monkeypatch):
    from astrai_b200.ops import backend

    monkeypatch.delenv("ASTR_BACKEND", raising=False)
    monkeypatch.delenv("ASTRAI_B200_ATTN", raising=False)
    assert backend.get_backend("cpu") is backend.ATTN_BACKEND.TORCH_NATIVE
    assert backend.get_backend("cuda") is backend.ATTN_BACKEND.TCGEN05 and not backend.explicit()
    assert backend.get_backend("cuda", use_default=False) is None
    with backend.attn_backend("torch_native"):
        assert backend.get_backend("cuda") is backend.ATTN_BACKEND.TORCH_NATIVE and backend.explicit()
        assert backend.get_backend("cuda", use_default=False) is backend.ATTN_BACKEND.TORCH_NATIVE
        with backend.attn_backend(backend.ATTN_BACKEND.TCGEN05):  # contexts nest and unwind
            assert backend.get_backend("cuda") is backend.ATTN_BACKEND.TCGEN05
        assert backend.get_backend("cuda") is backend.ATTN_BACKEND.TORCH_NATIVE
    assert backend.get_backend("cuda") is backend.ATTN_BACKEND.TCGEN05
    # the environment is a process-wide override: it wins over a context, as in the reference
    monkeypatch.setenv("ASTR_BACKEND", "torch_native")
    assert backend.get_backend("cuda") is backend.ATTN_BACKEND.TORCH_NATIVE and backend.explicit()
    with backend.attn_backend("cuda"):  # the reference's name for its kernel backend
        assert backend.get_backend("cuda") is backend.ATTN_BACKEND.TORCH_NATIVE
        assert backend.get_backend("cuda", use_default=False) is backend.ATTN_BACKEND.TORCH_NATIVE
    monkeypatch.delenv("ASTR_BACKEND")
    monkeypatch.setenv("ASTRAI_B200_ATTN", "sdpa")
    assert backend.get_backend("cuda") is backend.ATTN_BACKEND.TORCH_NATIVE
    monkeypatch.delenv("ASTRAI_B200_ATTN")
    with backend.attn_backend("cuda"):
        assert backend.get_backend("cuda") is backend.ATTN_BACKEND.TCGEN05
    with pytest.raises(ValueError):
        with backend.attn_backend("unknown"):
            pass
    assert backend.ATTN_BACKEND.parse("flash") is backend.ATTN_BACKEND.TCGEN05
    with pytest.raises(ValueError):
        backend.ATTN_BACKEND.parse("metal")
    assert backend.is_available("torch_native")


def test_every_public_name_of_the_reference_packages_exists_here():
    """The names the reference's packages export (their ``__all__`` lists, read once and written down here) resolve in the
    corresponding packages of this framework."""
    import importlib

    expected = {
        "astrai_b200.data": ["Streamable", "Recordable", "Store", "StoreFactory", "MmapStore", "JsonlStore", "DatasetFactory", "RDSampler"],
        "astrai_b200.inference": ["Executor", "InferenceEngine", "InferenceScheduler", "KVCache", "Task", "TaskManager", "sample"],
        "astrai_b200.tokenize": ["AutoTokenizer", "ChatTemplate", "MessageType", "Message", "Messages"],
        "astrai_b200.optim": ["composite_state_dict", "composite_step", "composite_zero_grad", "refresh_param_groups", "OptimizerFactory",
                              "Mano", "ManoAdamW", "MuonAdamW", "NAdamW", "Nora", "NoraNAdamW", "OptimizerParameterGroups", "nora_direction",
                              "nora_lr_scale", "partition_optimizer_parameters"],
        "astrai_b200.ops": ["ATTN_BACKEND", "AttentionBackend", "AttentionBackendFactory", "CudaBackend", "TorchNativeBackend",
                            "FlashAttnBackend", "TensorLayout", "attention", "attn_backend", "get_backend", "attn_decode", "attn_paged_decode",
                            "attn_prefill", "is_available", "KERNEL_NAMES", "apply_rotary_emb"],
        "astrai_b200.inference.network": ["FunctionDef", "ToolDef", "ChatCompletionRequest", "MessagesRequest", "ProtocolHandler"],
        "astrai_b200.models": ["apply_rotary_emb", "get_rotary_emb", "RotaryEmbedding", "AutoModel", "AutoRegressiveLM", "GQA", "MLA", "MLP",
                               "DeepSeekMoE"],
    }
    for module, names in expected.items():
        mod = importlib.import_module(module)
        missing = [n for n in names if not hasattr(mod, n)]
        assert not missing, (module, missing)
        assert set(names) <= set(mod.__all__), (module, sorted(set(names) - set(mod.__all__)))


def test_launch_strategy_is_chosen_from_the_environment(monkeypatch):
    from astrai_b200.parallel import LaunchStrategy, LocalStrategy, TorchrunStrategy, launch_strategy

    for name in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "LOCAL_WORLD_SIZE", "TORCHELASTIC_RUN_ID"):
        monkeypatch.delenv(name, raising=False)
    local = launch_strategy(1, backend="gloo", device_type="cpu")
    assert isinstance(local, LocalStrategy) and isinstance(local, LaunchStrategy) and local.master_port.isdigit()
    seen = {}
    local.launch(lambda **kw: seen.update(kw), value=3)  # a world of one runs in this process
    assert seen == {"value": 3}
    monkeypatch.setenv("RANK", "0")
    monkeypatch.setenv("WORLD_SIZE", "1")
    monkeypatch.setenv("MASTER_ADDR", "127.0.0.1")
    external = launch_strategy(1, backend="gloo", device_type="cpu", master_port="29733")
    assert isinstance(external, TorchrunStrategy) and external.master_port == "29733"
    with pytest.raises(NotImplementedError):
        LaunchStrategy(1, "gloo", "127.0.0.1", "1", "cpu").launch(print)
