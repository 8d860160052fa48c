"""HuggingFace -> native conversion: config fields, key renames, dense / MoE scoping, rejections, end-to-end load."""

import json

import pytest
import torch

from astrai_b200.serialization.hf import (
    HF_MODEL_TYPES, adapt_config, convert_hf_config, convert_hf_weights, looks_like_hf_state_dict,
)

LLAMA = dict(model_type="llama", vocab_size=128, hidden_size=16, num_hidden_layers=2, intermediate_size=32, rms_norm_eps=1e-5,
             tie_word_embeddings=False, max_position_embeddings=64, rope_theta=10000.0, num_attention_heads=4,
             num_key_value_heads=2)


def _cfg(**over):
    from astrai_b200.config import AutoRegressiveLMConfig

    return AutoRegressiveLMConfig.from_dict(convert_hf_config({**LLAMA, **over}))


def _hf_dense_state(layers=2, d=16, f=32, v=128, kv=8):
    sd = {"model.embed_tokens.weight": torch.randn(v, d), "model.norm.weight": torch.ones(d), "lm_head.weight": torch.randn(v, d)}
    for i in range(layers):
        p = f"model.layers.{i}."
        sd.update({p + "self_attn.q_proj.weight": torch.randn(d, d), p + "self_attn.k_proj.weight": torch.randn(kv, d),
                   p + "self_attn.v_proj.weight": torch.randn(kv, d), p + "self_attn.o_proj.weight": torch.randn(d, d),
                   p + "mlp.gate_proj.weight": torch.randn(f, d), p + "mlp.up_proj.weight": torch.randn(f, d),
                   p + "mlp.down_proj.weight": torch.randn(d, f), p + "input_layernorm.weight": torch.ones(d),
                   p + "post_attention_layernorm.weight": torch.ones(d)})
    return sd


def test_supported_families():
    assert {"llama", "mistral", "mixtral", "qwen2", "qwen2_moe", "gemma", "gemma2", "phi3"} == set(HF_MODEL_TYPES)


@pytest.mark.parametrize("family", sorted(HF_MODEL_TYPES))
def test_every_family_maps_the_common_fields(family):
    cfg = convert_hf_config({**LLAMA, "model_type": family})
    assert cfg["model_type"] == "autoregressive_lm" and cfg["hidden_size"] == 16 and cfg["num_key_value_heads"] == 2
    assert cfg["rope_theta"] == 10000.0 and cfg["rms_norm_eps"] == 1e-5


def test_native_configs_pass_through_untouched():
    raw = {"model_type": "autoregressive_lm", "hidden_size": 8}
    assert adapt_config(raw) is raw
    assert adapt_config({"hidden_size": 8}) == {"hidden_size": 8}


def test_missing_kv_heads_default_to_attention_heads():
    raw = dict(LLAMA)
    raw.pop("num_key_value_heads")
    assert convert_hf_config(raw)["num_key_value_heads"] == 4


def test_gemma_turns_on_qk_norm_and_explicit_flag_wins():
    assert convert_hf_config({**LLAMA, "model_type": "gemma2"})["use_qk_norm"] is True
    assert convert_hf_config({**LLAMA, "qk_norm": True})["use_qk_norm"] is True
    assert "use_qk_norm" not in convert_hf_config(LLAMA)


def test_bias_checkpoints_are_rejected():
    with pytest.raises(NotImplementedError, match="bias"):
        convert_hf_config({**LLAMA, "attention_bias": True})
    with pytest.raises(NotImplementedError, match="bias"):
        convert_hf_config({**LLAMA, "mlp_bias": True})


def test_explicit_head_dim_must_match_the_derived_one():
    assert convert_hf_config({**LLAMA, "head_dim": 4})["hidden_size"] == 16
    with pytest.raises(NotImplementedError, match="head_dim"):
        convert_hf_config({**LLAMA, "head_dim": 8})


def test_mixtral_style_moe_fields():
    cfg = convert_hf_config({**LLAMA, "model_type": "mixtral", "num_local_experts": 8, "num_experts_per_tok": 2})
    assert cfg["ffn_type"] == "moe" and cfg["n_routed_experts"] == 8 and cfg["n_activated_experts"] == 2
    assert cfg["n_shared_experts"] == 0 and cfg["moe_intermediate_size"] == 32


def test_first_k_dense_layers_become_mlp_only_layers():
    cfg = convert_hf_config({**LLAMA, "n_routed_experts": 4, "n_activated_experts": 2, "first_k_dense_replace": 1})
    assert cfg["mlp_only_layers"] == [0] and cfg["decoder_sparse_step"] == 1


def test_kv_lora_rank_selects_mla():
    assert convert_hf_config({**LLAMA, "kv_lora_rank": 8})["attn_type"] == "mla"


def test_hf_state_dict_detection():
    assert looks_like_hf_state_dict(_hf_dense_state())
    assert not looks_like_hf_state_dict({"layers.0.attention.q_proj.weight": 0, "embed_tokens.weight": 0})
    assert looks_like_hf_state_dict({"layers.0.mlp.experts.0.gate_proj.weight": 0})


def test_dense_keys_are_renamed_one_to_one():
    sd = _hf_dense_state()
    out = convert_hf_weights(sd, _cfg())
    assert len(out) == len(sd)
    for i in range(2):
        for leaf in ("attention.q_proj", "attention.k_proj", "attention.v_proj", "attention.o_proj", "mlp.gate", "mlp.up",
                     "mlp.down", "input_norm", "post_attention_norm"):
            assert f"layers.{i}.{leaf}.weight" in out
    assert {"embed_tokens.weight", "norm.weight", "lm_head.weight"} <= set(out)
    assert out["layers.1.mlp.down.weight"] is sd["model.layers.1.mlp.down_proj.weight"]  # renamed, not copied or permuted


def test_rotary_layout_is_not_permuted():
    sd = _hf_dense_state()
    out = convert_hf_weights(sd, _cfg())
    assert torch.equal(out["layers.0.attention.q_proj.weight"], sd["model.layers.0.self_attn.q_proj.weight"])


def test_native_keys_pass_through_and_unknown_keys_are_dropped(caplog):
    sd = {"layers.0.input_norm.weight": torch.ones(16), "model.layers.0.self_attn.rotary_emb.inv_freq": torch.ones(2)}
    with caplog.at_level("WARNING"):
        out = convert_hf_weights(sd, _cfg())
    assert list(out) == ["layers.0.input_norm.weight"] and "rotary_emb.inv_freq" in caplog.text


def test_moe_router_experts_and_shared_experts():
    cfg = _cfg(model_type="qwen2_moe", n_routed_experts=2, n_activated_experts=1, n_shared_experts=1)
    sd = {"model.layers.0.mlp.gate.weight": torch.randn(2, 16),
          "model.layers.0.mlp.experts.1.up_proj.weight": torch.randn(32, 16),
          "model.layers.0.mlp.shared_experts.0.down_proj.weight": torch.randn(16, 32),
          "model.layers.0.mlp.shared_expert.0.gate_proj.weight": torch.randn(32, 16)}
    out = convert_hf_weights(sd, cfg)
    assert set(out) == {"layers.0.mlp.router.weight", "layers.0.mlp.routed_experts.1.up.weight",
                        "layers.0.mlp.shared_experts.0.down.weight", "layers.0.mlp.shared_experts.0.gate.weight"}


def test_router_rule_only_applies_to_moe_models():
    out = convert_hf_weights({"model.layers.0.mlp.gate.weight": torch.randn(2, 16)}, _cfg())
    assert out == {}  # a dense model has no router: the key is unknown and dropped


def test_dense_layers_inside_a_moe_model_keep_their_mlp():
    cfg = _cfg(n_routed_experts=2, n_activated_experts=1, first_k_dense_replace=1)
    sd = {"model.layers.0.mlp.up_proj.weight": torch.randn(32, 16), "model.layers.1.mlp.up_proj.weight": torch.randn(32, 16)}
    out = convert_hf_weights(sd, cfg)
    assert list(out) == ["layers.0.mlp.up.weight"]  # layer 1 is sparse: a dense projection there has no destination


def test_deepseek_mla_checkpoints_are_rejected():
    cfg = _cfg(kv_lora_rank=8, qk_nope_head_dim=2, qk_rope_head_dim=2)
    with pytest.raises(NotImplementedError, match="MLA"):
        convert_hf_weights({"model.layers.0.self_attn.kv_a_proj_with_mqa.weight": torch.zeros(1)}, cfg)


def test_qk_norm_weights_are_renamed():
    out = convert_hf_weights({"model.layers.1.self_attn.q_norm.weight": torch.ones(4),
                              "model.layers.1.self_attn.k_norm.weight": torch.ones(4)}, _cfg(qk_norm=True))
    assert set(out) == {"layers.1.attention.q_norm.weight", "layers.1.attention.k_norm.weight"}


def test_from_pretrained_loads_an_hf_directory(tmp_path):
    from safetensors.torch import save_file

    from astrai_b200.models import AutoModel

    sd = _hf_dense_state()
    save_file({k: v.contiguous() for k, v in sd.items()}, str(tmp_path / "model.safetensors"))
    (tmp_path / "config.json").write_text(json.dumps(LLAMA))
    model = AutoModel.from_pretrained(str(tmp_path))
    assert torch.equal(model.layers[1].mlp.down.weight, sd["model.layers.1.mlp.down_proj.weight"])
    assert torch.equal(model.embed_tokens.weight, sd["model.embed_tokens.weight"])
    out = model(torch.randint(0, 128, (1, 8)))
    assert out["logits"].shape == (1, 8, 128) and torch.isfinite(out["logits"]).all()


def test_from_pretrained_loads_a_sharded_hf_directory(tmp_path):
    from safetensors.torch import save_file

    from astrai_b200.models import AutoModel

    sd = _hf_dense_state()
    keys = sorted(sd)
    halves = {"model-00001-of-00002.safetensors": keys[: len(keys) // 2], "model-00002-of-00002.safetensors": keys[len(keys) // 2:]}
    weight_map = {}
    for fname, ks in halves.items():
        save_file({k: sd[k].contiguous() for k in ks}, str(tmp_path / fname))
        weight_map.update({k: fname for k in ks})
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": weight_map}))
    (tmp_path / "config.json").write_text(json.dumps(LLAMA))
    model = AutoModel.from_pretrained(str(tmp_path))
    assert torch.equal(model.layers[0].attention.k_proj.weight, sd["model.layers.0.self_attn.k_proj.weight"])


def test_tied_hf_checkpoint_without_lm_head(tmp_path):
    from safetensors.torch import save_file

    from astrai_b200.models import AutoModel

    sd = _hf_dense_state()
    sd.pop("lm_head.weight")
    save_file({k: v.contiguous() for k, v in sd.items()}, str(tmp_path / "model.safetensors"))
    (tmp_path / "config.json").write_text(json.dumps({**LLAMA, "tie_word_embeddings": True}))
    model = AutoModel.from_pretrained(str(tmp_path))
    assert model.lm_head.weight is model.embed_tokens.weight
