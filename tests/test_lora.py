"""LoRA adapters: injection, forward equivalence, what trains, merge, adapter files, error paths."""

import json

import pytest
import torch

from helpers import tiny_config


def _model(**over):
    from astrai_b200.models import AutoRegressiveLM

    torch.manual_seed(0)
    return AutoRegressiveLM(tiny_config(**over))


def _lora_modules(model):
    from astrai_b200.models.lora import LoRALinear

    return {n: m for n, m in model.named_modules() if isinstance(m, LoRALinear)}


def test_default_targets_are_the_attention_projections():
    from astrai_b200.models.lora import inject_lora

    model = _model()
    cfg = inject_lora(model, r=4, alpha=8)
    names = _lora_modules(model)
    assert len(names) == 2 * 4 and all(n.rsplit(".", 1)[1] in ("q_proj", "k_proj", "v_proj", "o_proj") for n in names)
    assert set(cfg.target_modules) == {"q_proj", "k_proj", "v_proj", "o_proj"} and (cfg.r, cfg.alpha) == (4, 8)


def test_custom_targets_and_ffn_layers():
    from astrai_b200.models.lora import inject_lora

    model = _model()
    inject_lora(model, r=2, alpha=4, target_modules={"up", "down"})
    assert sorted({n.rsplit(".", 1)[1] for n in _lora_modules(model)}) == ["down", "up"]


def test_unknown_target_injects_nothing(caplog):
    from astrai_b200.models.lora import inject_lora

    model = _model()
    with caplog.at_level("WARNING"):
        inject_lora(model, target_modules={"does_not_exist"})
    assert not _lora_modules(model) and "No LoRA layers injected" in caplog.text


def test_fresh_adapter_leaves_the_function_unchanged():
    from astrai_b200.models.lora import inject_lora

    model = _model()
    ids = torch.randint(0, 1000, (2, 10))
    before = model(ids)["logits"]
    inject_lora(model, r=4, alpha=8)
    assert torch.allclose(model(ids)["logits"], before, atol=1e-6)  # B starts at zero


def test_only_adapter_parameters_train():
    from astrai_b200.models.lora import inject_lora

    model = _model()
    inject_lora(model, r=4, alpha=8, target_modules={"q_proj"})
    for name, p in model.named_parameters():
        wrapped_base = name.endswith("q_proj.weight")
        assert p.requires_grad == (not wrapped_base), name
    loss = model(torch.randint(0, 1000, (2, 10)))["logits"].float().pow(2).mean()
    loss.backward()
    mods = _lora_modules(model)
    assert all(m.lora_B.grad is not None and m.weight.grad is None for m in mods.values())


def test_shapes_scaling_and_init():
    from astrai_b200.models.layers import Linear
    from astrai_b200.models.lora import LoRALinear

    base = Linear(12, 20)
    base.reset_parameters() if hasattr(base, "reset_parameters") else None
    lora = LoRALinear(base, r=3, alpha=6)
    assert lora.lora_A.shape == (3, 12) and lora.lora_B.shape == (20, 3) and lora.scaling == 2.0
    assert torch.count_nonzero(lora.lora_B) == 0 and torch.count_nonzero(lora.lora_A) > 0
    assert lora.weight is base.weight


def test_adapter_contribution_is_scaled_low_rank_product():
    from astrai_b200.models.layers import Linear
    from astrai_b200.models.lora import LoRALinear

    torch.manual_seed(1)
    base = Linear(8, 6)
    torch.nn.init.normal_(base.weight, std=0.1)
    lora = LoRALinear(base, r=2, alpha=8)
    with torch.no_grad():
        lora.lora_B.normal_()
    x = torch.randn(5, 8)
    want = x @ base.weight.t() + (x @ lora.lora_A.t() @ lora.lora_B.t()) * 4.0
    assert torch.allclose(lora(x), want, atol=1e-5)


def test_merge_folds_the_adapter_into_the_weight():
    from astrai_b200.models.lora import inject_lora, merge_lora

    model = _model()
    inject_lora(model, r=4, alpha=8)
    with torch.no_grad():
        for m in _lora_modules(model).values():
            m.lora_B.normal_(std=0.05)
    ids = torch.randint(0, 1000, (2, 10))
    with_adapter = model(ids)["logits"]
    merge_lora(model)
    assert torch.allclose(model(ids)["logits"], with_adapter, atol=1e-4)
    mods = _lora_modules(model)
    assert all(not hasattr(m, "lora_A") for m in mods.values())
    merge_lora(model)  # merging twice is a no-op
    assert torch.allclose(model(ids)["logits"], with_adapter, atol=1e-4)


def test_merge_without_adapters_warns(caplog):
    from astrai_b200.models.lora import merge_lora

    with caplog.at_level("WARNING"):
        merge_lora(_model())
    assert "No LoRA layers to merge" in caplog.text


def test_adapter_files_round_trip(tmp_path):
    from astrai_b200.models.lora import inject_lora, load_lora, save_lora

    model = _model()
    cfg = inject_lora(model, r=4, alpha=8, target_modules={"q_proj", "v_proj"})
    with torch.no_grad():
        for m in _lora_modules(model).values():
            m.lora_B.normal_(std=0.05)
    save_lora(model, str(tmp_path), cfg)
    raw = json.loads((tmp_path / "adapter_config.json").read_text())
    assert raw["r"] == 4 and raw["alpha"] == 8 and sorted(raw["target_modules"]) == ["q_proj", "v_proj"]
    assert (tmp_path / "adapter_model.safetensors").stat().st_size > 0
    ids = torch.randint(0, 1000, (2, 10))
    want = model(ids)["logits"]
    fresh = _model()
    loaded = load_lora(fresh, str(tmp_path))  # injects by itself, then loads
    assert (loaded.r, loaded.alpha) == (4, 8) and torch.allclose(fresh(ids)["logits"], want, atol=1e-6)


def test_adapter_file_holds_only_adapter_tensors(tmp_path):
    from safetensors.torch import load_file

    from astrai_b200.models.lora import inject_lora, save_lora

    model = _model()
    cfg = inject_lora(model, r=2, alpha=4, target_modules={"o_proj"})
    save_lora(model, str(tmp_path), cfg)
    keys = list(load_file(str(tmp_path / "adapter_model.safetensors")))
    assert len(keys) == 2 * 2 and all(k.endswith((".lora_A", ".lora_B")) for k in keys)


def test_saving_a_model_without_adapters_fails(tmp_path):
    from astrai_b200.config.train_config import LoRAConfig
    from astrai_b200.models.lora import save_lora

    with pytest.raises(RuntimeError, match="No LoRA parameters"):
        save_lora(_model(), str(tmp_path), LoRAConfig())


def test_loading_onto_an_injected_model_does_not_wrap_twice(tmp_path, caplog):
    from astrai_b200.models.lora import inject_lora, load_lora, save_lora

    src = _model()
    cfg = inject_lora(src, r=4, alpha=8)
    save_lora(src, str(tmp_path), cfg)
    dst = _model()
    inject_lora(dst, r=4, alpha=8)
    with caplog.at_level("WARNING"):
        load_lora(dst, str(tmp_path))
    assert len(_lora_modules(dst)) == 8 and "already has LoRA layers" in caplog.text


def test_rank_mismatch_is_reported(tmp_path):
    from astrai_b200.models.lora import inject_lora, load_lora, save_lora

    src = _model()
    save_lora(src, str(tmp_path), inject_lora(src, r=4, alpha=8))
    dst = _model()
    inject_lora(dst, r=2, alpha=8)
    with pytest.raises(RuntimeError, match="shapes do not match"):
        load_lora(dst, str(tmp_path))


def test_state_dict_keys_of_an_injected_model():
    from astrai_b200.models.lora import inject_lora

    model = _model()
    inject_lora(model, r=2, alpha=4, target_modules={"q_proj"})
    keys = set(model.state_dict())
    assert "layers.0.attention.q_proj.weight" in keys  # the frozen base weight keeps its checkpoint key
    assert {"layers.0.attention.q_proj.lora_A", "layers.0.attention.q_proj.lora_B"} <= keys


def test_trainer_config_injects_adapters(tmp_path):
    from astrai_b200.config import TrainConfig
    from astrai_b200.config.train_config import LoRAConfig
    from astrai_b200.trainer.train_context import TrainContextBuilder
    from helpers import RandomTokens

    cfg = TrainConfig(model_fn=_model, strategy="seq", dataset=RandomTokens(8, 12),
                      optimizer_fn=lambda m: torch.optim.AdamW([p for p in m.parameters() if p.requires_grad], lr=1e-2),
                      batch_per_device=2, ckpt_dir=str(tmp_path), device_type="cpu", backend="gloo",
                      lora=LoRAConfig(r=2, alpha=4, target_modules=("q_proj", "v_proj")))
    ctx = TrainContextBuilder(cfg).build()
    assert len(_lora_modules(ctx.model)) == 4
    trainable = [n for n, p in ctx.model.named_parameters() if p.requires_grad]
    assert any(n.endswith("lora_A") for n in trainable) and not any(n.endswith("q_proj.weight") for n in trainable)
