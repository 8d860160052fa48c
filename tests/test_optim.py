"""Matrix optimizers, parameter partition, composite state dicts, fused AdamW on CPU."""

import math

import pytest
import torch

from helpers import tiny_config


def _model(**over):
    from astrai_b200.models import AutoRegressiveLM

    torch.manual_seed(0)
    return AutoRegressiveLM(tiny_config(**over))


def test_partition_by_module_role():
    from astrai_b200.optim import partition_optimizer_parameters

    m = _model(use_qk_norm=True)
    g = partition_optimizer_parameters(m)
    names = {id(p): n for n, p in m.named_parameters()}
    assert all(names[id(p)].endswith("_proj.weight") or ".mlp." in names[id(p)] for p in g.nora)
    plain = {names[id(p)] for p in g.nadamw_no_decay}
    assert "embed_tokens.weight" in plain and "lm_head.weight" in plain and "norm.weight" in plain
    assert "layers.0.attention.q_norm.weight" in plain
    total = len(g.nora) + len(g.nadamw_decay) + len(g.nadamw_no_decay)
    assert total == len(list(m.parameters()))


def test_nora_direction_is_tangent_and_unit():
    from astrai_b200.optim import nora_direction, nora_lr_scale

    torch.manual_seed(0)
    p, u = torch.randn(6, 9), torch.randn(6, 9)
    d = nora_direction(u, p)
    assert torch.allclose(d.norm(dim=-1), torch.ones(6), atol=1e-5)
    assert torch.allclose((d * p).sum(-1), torch.zeros(6), atol=1e-5)
    assert nora_lr_scale(1.0, (8, 2)) == 2.0 and nora_lr_scale(1.0, (2, 8)) == 1.0


def test_newton_schulz_orthogonalises():
    from astrai_b200.optim import newton_schulz

    torch.manual_seed(0)
    for shape in ((16, 32), (48, 16)):
        x = newton_schulz(torch.randn(*shape))
        s = torch.linalg.svdvals(x.float())
        assert s.max() < 1.3 and s.min() > 0.3  # singular values pushed toward one


@pytest.mark.parametrize("name", ["muon_adamw", "nora_nadamw", "mano_adamw", "fused_adamw"])
def test_optimizers_reduce_loss_and_roundtrip_state(name):
    from astrai_b200.optim import OptimizerFactory

    m = _model()
    opt = OptimizerFactory.create(name, m if name != "fused_adamw" else m.parameters(), lr=1e-2)
    ids = torch.randint(0, 1000, (2, 9))

    def loss_fn():
        return torch.nn.functional.cross_entropy(m(ids[:, :-1])["logits"].flatten(0, 1), ids[:, 1:].flatten())

    first = loss_fn().item()
    for _ in range(12):
        opt.zero_grad()
        loss = loss_fn()
        loss.backward()
        opt.step()
    assert loss.item() < first
    assert len(opt.param_groups) >= 1 and "lr" in opt.param_groups[-1]
    state = opt.state_dict()
    m2 = _model()
    opt2 = OptimizerFactory.create(name, m2 if name != "fused_adamw" else m2.parameters(), lr=1e-2)
    opt2.load_state_dict(state)
    if name == "nora_nadamw":
        with pytest.raises(ValueError):
            opt2.load_state_dict({"muon": None, "adamw": None})
    if name == "mano_adamw":
        with pytest.raises(ValueError):
            opt2.load_state_dict({"nora": None, "nadamw": None})


def test_mano_alternates_axes_and_matrix_only():
    from astrai_b200.optim import Mano, Nora

    p = torch.nn.Parameter(torch.randn(4, 6))
    opt = Mano([p], lr=0.1, weight_decay=0.0)
    p.grad = torch.randn(4, 6)
    opt.step()
    assert opt.param_groups[0]["steps"] == 1
    with pytest.raises(ValueError):
        Mano([torch.nn.Parameter(torch.randn(3))])
    with pytest.raises(ValueError):
        Nora([torch.nn.Parameter(torch.randn(3))])


def test_nadamw_matches_formula():
    from astrai_b200.optim import NAdamW

    p = torch.nn.Parameter(torch.tensor([1.0, -2.0]))
    opt = NAdamW([p], lr=0.1, betas=(0.9, 0.99), eps=1e-8, weight_decay=0.0)
    g = torch.tensor([0.5, 0.25])
    p.grad = g.clone()
    opt.step()
    m, v = 0.1 * g, 0.01 * g * g
    expect = torch.tensor([1.0, -2.0]) - 0.1 * ((0.9 * m + 0.1 * g) / 0.1) / ((v / 0.01).sqrt() + 1e-8)
    assert torch.allclose(p.detach(), expect, atol=1e-6)


def test_fused_adamw_cpu_matches_torch():
    from astrai_b200.optim import FusedAdamW

    torch.manual_seed(0)
    a = torch.nn.Parameter(torch.randn(10, 3))
    b = torch.nn.Parameter(a.detach().clone())
    ours = FusedAdamW([a], lr=1e-2, betas=(0.9, 0.95), weight_decay=0.1)
    ref = torch.optim.AdamW([b], lr=1e-2, betas=(0.9, 0.95), weight_decay=0.1)
    for _ in range(5):
        g = torch.randn(10, 3)
        a.grad, b.grad = g.clone(), g.clone()
        ours.step()
        ref.step()
    assert torch.allclose(a, b, atol=1e-6)
