"""Mixture-of-experts model structure and outputs, router diagnostics, encoder pooling, tied weights (behaviours the
reference checks in ``tests/module/test_forward_configs.py``, ``test_model_forward.py``, ``test_encoder.py`` and
``test_tie_weight.py``)."""

import math

import pytest
import torch

from helpers import tiny_config

MOE = dict(ffn_type="moe", n_routed_experts=4, n_shared_experts=1, n_activated_experts=2)


def _lm(**over):
    from astrai_b200.models import AutoRegressiveLM

    torch.manual_seed(0)
    return AutoRegressiveLM(tiny_config(**over))


def _kinds(model):
    return [type(layer.mlp).__name__ for layer in model.layers]


# ------------------------------------------------------------------------------------------------ layer structure
def test_every_layer_is_sparse_by_default():
    assert _kinds(_lm(num_hidden_layers=4, **MOE)) == ["DeepSeekMoE"] * 4
    assert _kinds(_lm(num_hidden_layers=3)) == ["MLP"] * 3


def test_sparse_step_and_dense_layer_list_pick_the_ffn_per_layer():
    assert _kinds(_lm(num_hidden_layers=4, decoder_sparse_step=2, **MOE)) == ["MLP", "DeepSeekMoE", "MLP", "DeepSeekMoE"]
    assert _kinds(_lm(num_hidden_layers=4, mlp_only_layers=[0, 3], **MOE)) == ["MLP", "DeepSeekMoE", "DeepSeekMoE", "MLP"]
    assert _kinds(_lm(num_hidden_layers=6, decoder_sparse_step=3, mlp_only_layers=[5], **MOE)) == ["MLP", "MLP", "DeepSeekMoE", "MLP", "MLP", "MLP"]


@pytest.mark.parametrize("step", [0, -1])
def test_invalid_sparse_step_is_rejected(step):
    with pytest.raises(Exception, match="decoder_sparse_step"):
        tiny_config(decoder_sparse_step=step, **MOE)


def test_expert_widths_follow_their_own_config_fields():
    m = _lm(intermediate_size=16, moe_intermediate_size=8, shared_expert_intermediate_size=24, **MOE)
    moe = m.layers[0].mlp
    assert moe.routed_experts[0].gate.weight.shape == (8, 8) and moe.routed_experts[0].down.weight.shape == (8, 8)
    assert moe.shared_experts[0].gate.weight.shape == (24, 8)
    assert moe.router.weight.shape == (4, 8) and len(moe.routed_experts) == 4 and len(moe.shared_experts) == 1
    default = _lm(intermediate_size=16, **MOE).layers[0].mlp
    assert default.routed_experts[0].gate.weight.shape == (16, 8) and default.shared_experts[0].gate.weight.shape == (16, 8)
    none_shared = _lm(**{**MOE, "n_shared_experts": 0}).layers[0].mlp
    assert len(none_shared.shared_experts) == 0


def test_incomplete_moe_config_fails_with_a_clear_message():
    with pytest.raises(ValueError, match="n_activated_experts"):
        _lm(ffn_type="moe", n_routed_experts=4)


# ------------------------------------------------------------------------------------------------------- routing
def test_routing_weights_are_normalised_unless_switched_off():
    x = torch.randn(10, 8)
    norm = _lm(**MOE).layers[0].mlp
    w, idx, _, _ = norm.route(x, False)
    assert torch.allclose(w.sum(-1), torch.ones(10), atol=1e-6) and idx.shape == (10, 2)
    raw = _lm(norm_topk_prob=False, **MOE).layers[0].mlp
    w2, idx2, _, _ = raw.route(x, False)
    assert (w2.sum(-1) < 1.0).all()  # plain softmax mass of the two chosen experts
    assert (idx2[:, 0] != idx2[:, 1]).all()


def test_moe_layer_equals_a_dense_sum_over_chosen_experts():
    moe = _lm(**MOE).layers[0].mlp.eval()
    x = torch.randn(6, 8)
    out = moe(x)
    assert out["aux_loss"] is None and out["router_stats"] is None  # nothing to regularise in eval mode
    w, idx, _, _ = moe.route(x, False)
    want = torch.zeros_like(x)
    for t in range(6):
        for j in range(2):
            want[t] += w[t, j] * moe.routed_experts[int(idx[t, j])](x[t:t + 1])["hidden_states"][0]
        want[t] += moe.shared_experts[0](x[t:t + 1])["hidden_states"][0]
    assert torch.allclose(out["hidden_states"], want, atol=1e-5)
    assert moe(x.view(2, 3, 8))["hidden_states"].shape == (2, 3, 8)


def test_aux_loss_and_router_stats_only_while_training_with_grad():
    m = _lm(**MOE)
    ids = torch.randint(0, 1000, (2, 9))
    m.train()
    out = m(ids)
    assert out["aux_loss"].ndim == 0 and out["aux_loss"] > 0 and len(out["router_stats"]) == 2
    stats = out["router_stats"][0]
    assert stats["probs"].shape == (18, 4) and stats["topk_indices"].shape == (18, 2) and not stats["probs"].requires_grad
    with torch.no_grad():
        assert "aux_loss" not in m(ids)
    m.eval()
    assert "aux_loss" not in m(ids) and "router_stats" not in m(ids)
    dense = _lm().train()
    assert "aux_loss" not in dense(ids)


def test_aux_loss_is_one_for_uniform_routing_and_grows_with_collapse():
    moe = _lm(**MOE).layers[0].mlp.train()
    with torch.no_grad():
        moe.router.weight.zero_()  # uniform probabilities: load x importance sums to 1 / E per expert
    _, _, aux, _ = moe.route(torch.randn(64, 8), True)
    assert float(aux.detach()) == pytest.approx(1.0, abs=0.02)
    with torch.no_grad():
        moe.router.weight[0] = 5.0  # expert 0 wins for inputs with a positive sum
    x = torch.rand(64, 8) + 0.5
    _, idx, aux2, _ = moe.route(x, True)
    assert (idx == 0).any(-1).all() and float(aux2.detach()) > 1.2


# ---------------------------------------------------------------------------------------------------- diagnostics
def test_diagnostics_of_uniform_and_collapsed_routers():
    from astrai_b200.trainer.strategy import moe_diagnostics

    assert moe_diagnostics([]) == {} and moe_diagnostics(None) == {}
    e, n = 4, 16
    uniform = {"probs": torch.full((n, e), 1.0 / e), "topk_indices": torch.arange(n * 2).reshape(n, 2) % e}
    d = {k: float(v) for k, v in moe_diagnostics([uniform]).items()}
    assert set(d) == {"router_entropy", "dead_expert_fraction", "load_imbalance_mean", "load_imbalance_max"}
    assert d["router_entropy"] == pytest.approx(math.log(e), abs=1e-5)  # the most a router over four experts can have
    assert d["dead_expert_fraction"] == 0.0 and d["load_imbalance_mean"] == pytest.approx(0.0) and d["load_imbalance_max"] == pytest.approx(1.0)
    onehot = torch.zeros(n, e)
    onehot[:, 0] = 1.0
    collapsed = {"probs": onehot, "topk_indices": torch.zeros(n, 2, dtype=torch.long)}
    c = {k: float(v) for k, v in moe_diagnostics([collapsed]).items()}
    assert c["router_entropy"] == pytest.approx(0.0, abs=1e-5) and c["dead_expert_fraction"] == 0.75 and c["load_imbalance_max"] == pytest.approx(4.0)
    both = {k: float(v) for k, v in moe_diagnostics([uniform, collapsed]).items()}
    assert both["dead_expert_fraction"] == pytest.approx(0.375)  # the mean over layers


def test_diagnostics_flow_from_a_wrapped_model_into_the_strategy():
    from astrai_b200.trainer import StrategyFactory

    class Wrapper(torch.nn.Module):  # a stand-in for a parallel wrapper: forwards everything to the inner module
        def __init__(self, inner):
            super().__init__()
            self.module = inner

        def forward(self, *a, **k):
            return self.module(*a, **k)

    model = Wrapper(_lm(**MOE)).train()
    ids = torch.randint(0, 1000, (2, 11))
    s = StrategyFactory.create("seq", model=model, device="cpu")
    s({"input_ids": ids[:, :-1], "target_ids": ids[:, 1:]})
    got = s._moe_metrics.resolved()
    assert {"router_entropy", "dead_expert_fraction", "load_imbalance_mean", "load_imbalance_max", "aux_loss"} <= set(got)
    sft = StrategyFactory.create("sft", model=model, device="cpu", moe_aux_loss_coef=0.0)
    out = sft({"input_ids": ids[:, :-1], "target_ids": ids[:, 1:], "loss_mask": torch.ones(2, 10, dtype=torch.bool),
               "position_ids": torch.arange(10).repeat(2, 1)})
    assert out["metrics"].resolved()["moe_aux_loss_weighted"] == 0.0


# -------------------------------------------------------------------------------------------------------- encoder
@pytest.mark.parametrize("pooling", ["mean", "cls", "last"])
def test_encoder_pooling_modes(pooling):
    from astrai_b200.config import EncoderConfig
    from astrai_b200.models import EmbeddingEncoder

    from helpers import TINY

    torch.manual_seed(0)
    cfg = EncoderConfig(**{k: v for k, v in TINY.items() if k != "tie_word_embeddings"}, pooling_type=pooling, normalize_embeddings=False)
    enc = EmbeddingEncoder(cfg).eval()
    ids = torch.randint(1, 1000, (3, 7))
    mask = torch.ones(3, 7, dtype=torch.bool)
    mask[1, 4:] = False
    out = enc(ids, mask)
    emb = out["embeddings"] if isinstance(out, dict) else out
    assert emb.shape == (3, 8) and torch.isfinite(emb).all()
    changed = ids.clone()
    changed[1, 5] = (changed[1, 5] + 1) % 1000  # a padded position
    emb2 = enc(changed, mask)
    emb2 = emb2["embeddings"] if isinstance(emb2, dict) else emb2
    assert torch.allclose(emb[1], emb2[1], atol=1e-6)  # padding never reaches the pooled vector


def test_encoder_normalisation_gives_unit_vectors():
    from astrai_b200.config import EncoderConfig
    from astrai_b200.models import EmbeddingEncoder

    from helpers import TINY

    cfg = EncoderConfig(**{k: v for k, v in TINY.items() if k != "tie_word_embeddings"}, pooling_type="mean", normalize_embeddings=True)
    out = EmbeddingEncoder(cfg).eval()(torch.randint(1, 1000, (4, 6)), torch.ones(4, 6, dtype=torch.bool))
    emb = out["embeddings"] if isinstance(out, dict) else out
    assert torch.allclose(emb.norm(dim=-1), torch.ones(4), atol=1e-5)


# ---------------------------------------------------------------------------------------------------- tied weights
def test_tied_head_shares_storage_and_survives_save_and_load(tmp_path):
    from astrai_b200.models import AutoModel

    m = _lm(tie_word_embeddings=True)
    assert m.lm_head.weight is m.embed_tokens.weight or m.lm_head.weight.data_ptr() == m.embed_tokens.weight.data_ptr()
    assert "lm_head.weight" not in m.state_dict()
    m.save_pretrained(tmp_path / "tied")
    back = AutoModel.from_pretrained(tmp_path / "tied")
    assert back.lm_head.weight.data_ptr() == back.embed_tokens.weight.data_ptr()
    ids = torch.randint(0, 1000, (1, 5))
    assert torch.allclose(m.eval()(ids)["logits"], back.eval()(ids)["logits"], atol=1e-6)
    with torch.no_grad():
        back.embed_tokens.weight[3] += 1.0
    assert torch.equal(back.lm_head.weight[3], back.embed_tokens.weight[3])  # one tensor, two roles
    untied = _lm(tie_word_embeddings=False)
    assert untied.lm_head.weight.data_ptr() != untied.embed_tokens.weight.data_ptr() and "lm_head.weight" in untied.state_dict()


def test_untied_model_loads_a_checkpoint_without_a_head():
    tied, untied = _lm(tie_word_embeddings=True), _lm(tie_word_embeddings=False)
    untied.load_state_dict(tied.state_dict())  # the head is initialised from the embedding, as a copy
    assert torch.equal(untied.lm_head.weight, untied.embed_tokens.weight)
    assert untied.lm_head.weight.data_ptr() != untied.embed_tokens.weight.data_ptr()
