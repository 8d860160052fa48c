"""Model zoo on the CPU oracle path: shapes, configs, state-dict layout, parity with the reference package."""

import os
import sys

import pytest
import torch

from helpers import tiny_config

CONFIGS = [
    dict(),
    dict(tie_word_embeddings=True),
    dict(use_qk_norm=True, use_gated_attention=True),
    dict(attn_type="mla", kv_lora_rank=4, qk_nope_head_dim=2, qk_rope_head_dim=2),
    dict(attn_type="mla", kv_lora_rank=4, qk_nope_head_dim=2, qk_rope_head_dim=2, q_lora_rank=6, use_qk_norm=True),
    dict(ffn_type="moe", n_routed_experts=4, n_shared_experts=1, n_activated_experts=2, moe_intermediate_size=8),
    dict(ffn_type="moe", n_routed_experts=4, n_shared_experts=0, n_activated_experts=2, decoder_sparse_step=2),
    dict(ffn_type="moe", n_routed_experts=4, n_shared_experts=2, n_activated_experts=1, mlp_only_layers=[0], norm_topk_prob=False),
    dict(rope_theta=500000.0, rope_scaling={"type": "ntk", "factor": 2.0}),
    dict(num_key_value_heads=2),
]


@pytest.mark.parametrize("over", CONFIGS)
def test_forward_configs(over):
    from astrai_b200.models import AutoRegressiveLM

    torch.manual_seed(0)
    m = AutoRegressiveLM(tiny_config(**over))
    ids = torch.randint(0, 1000, (2, 12))
    out = m(ids)
    assert out["logits"].shape == (2, 12, 1000) and torch.isfinite(out["logits"]).all()
    if over.get("ffn_type") == "moe":
        m.train()
        out = m(ids)
        assert out["aux_loss"].ndim == 0 and len(out["router_stats"]) >= 1
        out["logits"].sum().backward()
    pad = torch.ones(2, 12, dtype=torch.bool)
    pad[1, 8:] = False
    assert torch.isfinite(m(ids, pad)["logits"]).all()


def test_forward_contract_errors():
    from astrai_b200.models import AutoRegressiveLM

    m = AutoRegressiveLM(tiny_config())
    with pytest.raises(ValueError):
        m(torch.zeros(5, dtype=torch.long))
    with pytest.raises(ValueError):
        m(torch.zeros(1, 5, dtype=torch.long), kv_cache=object())
    with pytest.raises(ValueError):
        m(torch.zeros(1, 5, dtype=torch.long), fwd="prefill")
    with pytest.raises(ValueError):
        m(torch.zeros(5, dtype=torch.long), fwd="bogus", kv_cache=object())


def test_padding_mask_is_not_causal():
    """A 2-D mask makes the pass bidirectional over valid keys (reference quirk)."""
    from astrai_b200.models import AutoRegressiveLM

    torch.manual_seed(0)
    m = AutoRegressiveLM(tiny_config()).eval()
    ids = torch.randint(0, 1000, (1, 8))
    ids2 = ids.clone()
    ids2[0, -1] = (ids2[0, -1] + 1) % 1000
    full = torch.ones(1, 8, dtype=torch.bool)
    a, b = m(ids, full)["logits"], m(ids2, full)["logits"]
    assert not torch.allclose(a[0, 0], b[0, 0])  # position 0 sees the last token
    a, b = m(ids)["logits"], m(ids2)["logits"]
    assert torch.allclose(a[0, 0], b[0, 0])  # causal without a mask


def test_tied_weights_state_dict():
    from astrai_b200.models import AutoRegressiveLM

    m = AutoRegressiveLM(tiny_config(tie_word_embeddings=True))
    assert m.lm_head.weight is m.embed_tokens.weight
    sd = m.state_dict()
    assert "lm_head.weight" not in sd and "embed_tokens.weight" in sd
    m2 = AutoRegressiveLM(tiny_config(tie_word_embeddings=True))
    m2.load_state_dict(sd)
    assert torch.equal(m2.lm_head.weight, m.embed_tokens.weight)
    untied = AutoRegressiveLM(tiny_config())
    untied.load_state_dict(sd)  # missing head is cloned from the embedding
    assert torch.equal(untied.lm_head.weight, sd["embed_tokens.weight"])
    assert untied.lm_head.weight is not untied.embed_tokens.weight


def test_state_dict_key_layout():
    from astrai_b200.models import AutoRegressiveLM

    keys = set(AutoRegressiveLM(tiny_config(use_qk_norm=True, use_gated_attention=True)).state_dict())
    for k in ("embed_tokens.weight", "norm.weight", "lm_head.weight", "layers.0.input_norm.weight",
              "layers.0.post_attention_norm.weight", "layers.1.attention.q_proj.weight", "layers.1.attention.o_proj.weight",
              "layers.0.attention.q_norm.weight", "layers.0.attention.gate.weight", "layers.0.mlp.up.weight",
              "layers.0.mlp.gate.weight", "layers.0.mlp.down.weight"):
        assert k in keys
    moe = set(AutoRegressiveLM(tiny_config(ffn_type="moe", n_routed_experts=2, n_shared_experts=1, n_activated_experts=1)).state_dict())
    assert {"layers.0.mlp.router.weight", "layers.0.mlp.routed_experts.1.down.weight", "layers.0.mlp.shared_experts.0.up.weight"} <= moe
    mla = set(AutoRegressiveLM(tiny_config(attn_type="mla", kv_lora_rank=4, qk_nope_head_dim=2, qk_rope_head_dim=2)).state_dict())
    assert {"layers.0.attention.kv_a_proj.weight", "layers.0.attention.kv_norm.weight", "layers.0.attention.kv_b_proj.weight"} <= mla


def test_save_and_from_pretrained(tmp_path):
    from astrai_b200.models import AutoModel, AutoRegressiveLM

    m = AutoRegressiveLM(tiny_config(tie_word_embeddings=True)).eval()
    m.save_pretrained(tmp_path)
    assert (tmp_path / "config.json").exists() and (tmp_path / "model.safetensors").exists()
    m2 = AutoModel.from_pretrained(tmp_path).eval()
    ids = torch.randint(0, 1000, (1, 6))
    assert torch.equal(m(ids)["logits"], m2(ids)["logits"])


def test_init_std_rules():
    from astrai_b200.models import AutoRegressiveLM

    torch.manual_seed(0)
    m = AutoRegressiveLM(tiny_config(hidden_size=64, intermediate_size=256, num_hidden_layers=8, num_attention_heads=4, num_key_value_heads=4))
    assert abs(m.layers[0].attention.q_proj.weight.std().item() - 0.02) < 0.004
    assert abs(m.layers[0].attention.o_proj.weight.std().item() - 0.02 / 4) < 0.002
    assert abs(m.layers[0].mlp.down.weight.std().item() - 0.02 / 4) < 0.002
    assert torch.all(m.norm.weight == 1)


def test_encoder_pooling():
    from astrai_b200.config import EncoderConfig
    from astrai_b200.models import EmbeddingEncoder

    base = {k: v for k, v in tiny_config().to_dict().items() if k in EncoderConfig.__dataclass_fields__}
    ids = torch.randint(0, 1000, (3, 7))
    mask = torch.ones(3, 7, dtype=torch.bool)
    mask[0, 4:] = False
    for pooling in ("mean", "cls", "last"):
        enc = EmbeddingEncoder(EncoderConfig(**{**base, "model_type": "embedding", "pooling_type": pooling, "normalize_embeddings": True})).eval()
        out = enc(ids, mask)
        assert out.shape == (3, 8)
        assert torch.allclose(out.norm(dim=-1), torch.ones(3), atol=1e-5)


def test_lora_inject_merge_save_load(tmp_path):
    from astrai_b200.models import AutoRegressiveLM, inject_lora, load_lora, merge_lora, save_lora
    from astrai_b200.models.lora import LoRALinear

    torch.manual_seed(0)
    m = AutoRegressiveLM(tiny_config()).eval()
    ids = torch.randint(0, 1000, (1, 5))
    before = m(ids)["logits"]
    cfg = inject_lora(m, r=2, alpha=4, target_modules={"q_proj", "v_proj"})
    assert isinstance(m.layers[0].attention.q_proj, LoRALinear) and not isinstance(m.layers[0].attention.k_proj, LoRALinear)
    assert torch.allclose(m(ids)["logits"], before)  # B = 0 at injection
    assert not m.layers[0].attention.q_proj.weight.requires_grad
    with torch.no_grad():
        for mod in m.modules():
            if isinstance(mod, LoRALinear):
                mod.lora_B.normal_()
    changed = m(ids)["logits"]
    assert not torch.allclose(changed, before)
    save_lora(m, tmp_path, cfg)
    fresh = AutoRegressiveLM(tiny_config()).eval()
    fresh.load_state_dict({k: v for k, v in m.state_dict().items() if "lora" not in k})
    load_lora(fresh, tmp_path)
    assert torch.allclose(fresh(ids)["logits"], changed, atol=1e-6)
    merge_lora(m)
    assert torch.allclose(m(ids)["logits"], changed, atol=1e-5)
    assert not any(k.endswith("lora_A") for k in m.state_dict())


def test_logits_match_reference_package():
    """Same weights -> same logits as the unmodified reference model (when its install is present)."""
    ref_root = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_root, "astrai")):
        pytest.skip("reference package not installed")
    sys.path.insert(0, ref_root)
    try:
        from astrai.config import AutoRegressiveLMConfig as RefCfg
        from astrai.model import AutoRegressiveLM as RefLM
    finally:
        sys.path.remove(ref_root)
    from astrai_b200.models import AutoRegressiveLM

    for over in (dict(), dict(use_qk_norm=True, use_gated_attention=True),
                 dict(attn_type="mla", kv_lora_rank=4, qk_nope_head_dim=2, qk_rope_head_dim=2),
                 dict(ffn_type="moe", n_routed_experts=4, n_shared_experts=1, n_activated_experts=2)):
        cfg = tiny_config(**over)
        torch.manual_seed(0)
        ours = AutoRegressiveLM(cfg).eval()
        ref = RefLM(RefCfg(**cfg.to_dict())).eval()
        ref.load_state_dict(ours.state_dict())
        ids = torch.randint(0, 1000, (2, 10))
        with torch.no_grad():
            assert torch.allclose(ours(ids)["logits"], ref(ids)["logits"], atol=1e-5), over
