"""Update rules of the matrix optimizers one step at a time, the parameter partition over every model structure, the
composites' closure / scheduler / resume behaviour (behaviours the reference checks in ``tests/optim/test_nora_nadamw.py``
and ``tests/optim/test_mano_adamw.py``)."""

import copy
import math

import pytest
import torch

from helpers import tiny_config


def _model(**over):
    from astrai_b200.models import AutoRegressiveLM

    torch.manual_seed(0)
    return AutoRegressiveLM(tiny_config(**over))


# ------------------------------------------------------------------------------------------------------------ Nora
def test_nora_first_step_moves_every_row_by_the_learning_rate_along_its_tangent():
    from astrai_b200.optim import Nora

    torch.manual_seed(1)
    p = torch.nn.Parameter(torch.randn(5, 7))
    before = p.detach().clone()
    g = torch.randn(5, 7)
    p.grad = g.clone()
    Nora([p], lr=0.01, weight_decay=0.0).step()
    step = p.detach() - before
    assert torch.allclose(step.norm(dim=-1), torch.full((5,), 0.01), atol=1e-6)  # wide matrix: no extra scale
    unit = before / before.norm(dim=-1, keepdim=True)
    assert torch.allclose((step * unit).sum(-1), torch.zeros(5), atol=1e-7)      # no radial component
    assert ((step * g).sum(-1) < 0).all()                                        # and downhill


def test_nora_zero_gradient_rows_and_purely_radial_gradients_do_not_blow_up():
    from astrai_b200.optim import Nora

    p = torch.nn.Parameter(torch.tensor([[1.0, 0.0, 0.0], [0.0, 2.0, 0.0]]))
    p.grad = torch.tensor([[0.0, 0.0, 0.0], [0.0, 3.0, 0.0]])  # row 0: nothing; row 1: along the parameter row itself
    Nora([p], lr=0.1, weight_decay=0.0).step()
    assert torch.isfinite(p).all()
    assert torch.allclose(p.detach(), torch.tensor([[1.0, 0.0, 0.0], [0.0, 2.0, 0.0]]), atol=1e-5)


def test_nora_scales_the_step_for_tall_matrices_only():
    from astrai_b200.optim import nora_lr_scale

    assert nora_lr_scale(0.01, (64, 16)) == pytest.approx(0.02)
    assert nora_lr_scale(0.01, (16, 64)) == pytest.approx(0.01) and nora_lr_scale(0.01, (16, 16)) == pytest.approx(0.01)


def test_nora_weight_decay_shrinks_before_the_step():
    from astrai_b200.optim import Nora

    p = torch.nn.Parameter(torch.ones(2, 4))
    p.grad = torch.zeros(2, 4)
    Nora([p], lr=0.1, weight_decay=0.5).step()
    assert torch.allclose(p.detach(), torch.full((2, 4), 0.95), atol=1e-6)


@pytest.mark.parametrize("bad", [dict(lr=-1.0), dict(momentum=1.5), dict(beta=1.0), dict(eps=0.0), dict(weight_decay=-0.1)])
def test_nora_rejects_bad_hyperparameters(bad):
    from astrai_b200.optim import Nora

    with pytest.raises(ValueError):
        Nora([torch.nn.Parameter(torch.randn(2, 2))], **bad)


# ------------------------------------------------------------------------------------------------------------ Mano
def test_mano_step_follows_its_formula_on_alternating_axes():
    """``u - <u, p> p`` along the step's axis (columns on even steps, rows on odd ones), normalised along that axis and
    scaled by ``0.2 sqrt(n)``: every column (or row) moves by exactly that length."""
    from astrai_b200.optim import Mano

    torch.manual_seed(2)
    p = torch.nn.Parameter(torch.randn(4, 6))
    opt = Mano([p], lr=0.1, weight_decay=0.0, nesterov=False, momentum=0.0)
    for step, axis in ((0, 0), (1, 1), (2, 0)):
        before = p.detach().clone()
        g = torch.randn(4, 6)
        p.grad = g.clone()
        opt.step()
        tangent = g - (g * before).sum(dim=axis, keepdim=True) * before
        direction = tangent / (tangent.norm(dim=axis, keepdim=True) + 1e-8)
        scale = 0.1 * 0.2 * math.sqrt(before.shape[axis])
        assert torch.allclose(p.detach(), before - scale * direction, atol=1e-6), step
        delta = p.detach() - before
        assert torch.allclose(delta.norm(dim=axis), torch.full((before.shape[1 - axis],), scale), atol=1e-5), step
    assert opt.param_groups[0]["steps"] == 3


def test_mano_state_carries_the_axis_counter_through_a_resume():
    from astrai_b200.optim import Mano

    torch.manual_seed(3)
    a = torch.nn.Parameter(torch.randn(3, 5))
    b = torch.nn.Parameter(a.detach().clone())
    grads = [torch.randn(3, 5) for _ in range(4)]
    one = Mano([a], lr=0.05)
    for g in grads:
        a.grad = g.clone()
        one.step()
    two = Mano([b], lr=0.05)
    for g in grads[:2]:
        b.grad = g.clone()
        two.step()
    saved = copy.deepcopy(two.state_dict())
    resumed = Mano([b], lr=0.05)
    resumed.load_state_dict(saved)
    for g in grads[2:]:
        b.grad = g.clone()
        resumed.step()
    assert torch.allclose(a, b, atol=1e-6)


# ---------------------------------------------------------------------------------------------------------- NAdamW
def test_nadamw_two_steps_match_the_written_out_recursion():
    from astrai_b200.optim import NAdamW

    lr, b1, b2, eps, wd = 0.05, 0.9, 0.99, 1e-8, 0.1
    p = torch.nn.Parameter(torch.tensor([0.5, -1.5, 2.0]))
    opt = NAdamW([p], lr=lr, betas=(b1, b2), eps=eps, weight_decay=wd)
    x = p.detach().clone().double()
    m = v = torch.zeros(3, dtype=torch.double)
    for t, g in enumerate([torch.tensor([0.1, -0.2, 0.3]), torch.tensor([-0.4, 0.1, 0.2])], 1):
        p.grad = g.clone()
        opt.step()
        g = g.double()
        m = b1 * m + (1 - b1) * g
        v = b2 * v + (1 - b2) * g * g
        x = x * (1 - lr * wd)
        x = x - lr * ((b1 * m + (1 - b1) * g) / (1 - b1 ** t)) / ((v / (1 - b2 ** t)).sqrt() + eps)
    assert torch.allclose(p.detach().double(), x, atol=1e-6)


# ------------------------------------------------------------------------------------------------------- partition
STRUCTURES = [dict(), dict(tie_word_embeddings=True), dict(use_qk_norm=True, use_gated_attention=True),
              dict(attn_type="mla", kv_lora_rank=4, qk_nope_head_dim=2, qk_rope_head_dim=2, q_lora_rank=6),
              dict(ffn_type="moe", n_routed_experts=4, n_shared_experts=1, n_activated_experts=2)]


@pytest.mark.parametrize("over", STRUCTURES)
def test_partition_is_complete_and_disjoint_for_every_structure(over):
    from astrai_b200.optim import partition_optimizer_parameters

    m = _model(**over)
    g = partition_optimizer_parameters(m)
    groups = [g.nora, g.nadamw_decay, g.nadamw_no_decay]
    ids = [id(p) for grp in groups for p in grp]
    assert len(ids) == len(set(ids)) == len({id(p) for p in m.parameters()})  # every parameter once (a tied head counts once)
    assert all(p.ndim == 2 for p in g.nora)
    names = {id(p): n for n, p in m.named_parameters()}
    assert all("embed_tokens" not in names[id(p)] and "lm_head" not in names[id(p)] and "norm" not in names[id(p)] for p in g.nora)
    assert all(p.ndim < 2 or "embed" in names[id(p)] or "lm_head" in names[id(p)] or "router" in names[id(p)] or "norm" in names[id(p)]
               for p in g.nadamw_no_decay + g.nadamw_decay)


def test_factory_names_and_the_legacy_alias():
    from astrai_b200.optim import ManoAdamW, MuonAdamW, NoraNAdamW, OptimizerFactory

    assert OptimizerFactory._entries["nora_nadamw"] is NoraNAdamW and OptimizerFactory._entries["mano_adamw"] is ManoAdamW
    assert OptimizerFactory._entries["muon_adamw"] is MuonAdamW
    with pytest.raises((KeyError, ValueError)):
        OptimizerFactory.create("sgd_magic", _model())


# ------------------------------------------------------------------------------------------------------ composites
@pytest.mark.parametrize("name", ["nora_nadamw", "mano_adamw", "muon_adamw"])
def test_composites_run_a_closure_exactly_once_and_return_its_loss(name):
    from astrai_b200.optim import OptimizerFactory

    m = _model()
    opt = OptimizerFactory.create(name, m, lr=1e-3)
    ids = torch.randint(0, 1000, (2, 7))
    calls = []

    def closure():
        calls.append(1)
        opt.zero_grad()
        loss = m(ids)["logits"].float().pow(2).mean()
        loss.backward()
        return loss

    loss = opt.step(closure)
    assert len(calls) == 1 and loss is not None and torch.isfinite(loss)


def test_a_scheduler_scales_both_parts_of_a_composite_alike():
    from astrai_b200.optim import OptimizerFactory
    from astrai_b200.trainer import SchedulerFactory

    opt = OptimizerFactory.create("nora_nadamw", _model(), lr=3e-4, nora_lr=6e-3)
    base = [g["lr"] for g in opt.param_groups]
    assert max(base) == pytest.approx(6e-3) and min(base) == pytest.approx(3e-4)
    sched = SchedulerFactory.create("cosine", opt, warmup_steps=2, lr_decay_steps=10)
    ratios = []
    for _ in range(6):
        opt.step()
        sched.step()
        lrs = [g["lr"] for g in opt.param_groups]
        ratios.append(max(lrs) / min(lrs))
    assert all(r == pytest.approx(20.0, rel=1e-6) for r in ratios)  # the matrix : vector learning-rate ratio never drifts


@pytest.mark.parametrize("name", ["nora_nadamw", "mano_adamw"])
def test_resumed_composite_and_scheduler_continue_like_the_uninterrupted_run(name):
    from astrai_b200.optim import OptimizerFactory
    from astrai_b200.trainer import SchedulerFactory

    ids = [torch.randint(0, 1000, (2, 7), generator=torch.Generator().manual_seed(s)) for s in range(4)]

    def train(model, opt, sched, batches):
        for b in batches:
            opt.zero_grad()
            torch.nn.functional.cross_entropy(model(b[:, :-1])["logits"].flatten(0, 1), b[:, 1:].flatten()).backward()
            opt.step()
            sched.step()

    def build():
        m = _model()
        o = OptimizerFactory.create(name, m, lr=1e-2)
        return m, o, SchedulerFactory.create("cosine", o, warmup_steps=1, lr_decay_steps=8)

    m1, o1, s1 = build()
    train(m1, o1, s1, ids)
    m2, o2, s2 = build()
    train(m2, o2, s2, ids[:2])
    saved = copy.deepcopy((m2.state_dict(), o2.state_dict(), s2.state_dict()))
    m3, o3, s3 = build()
    m3.load_state_dict(saved[0])
    o3.load_state_dict(saved[1])
    s3.load_state_dict(saved[2])
    train(m3, o3, s3, ids[2:])
    for a, b in zip(m1.parameters(), m3.parameters()):
        assert torch.allclose(a, b, atol=1e-6)
    assert [g["lr"] for g in o1.param_groups] == pytest.approx([g["lr"] for g in o3.param_groups])


def test_composites_refuse_each_others_checkpoints():
    from astrai_b200.optim import OptimizerFactory

    nora = OptimizerFactory.create("nora_nadamw", _model())
    mano = OptimizerFactory.create("mano_adamw", _model())
    muon = OptimizerFactory.create("muon_adamw", _model())
    with pytest.raises(ValueError):
        nora.load_state_dict(muon.state_dict())
    with pytest.raises(ValueError):
        mano.load_state_dict(nora.state_dict())
    nora.load_state_dict(copy.deepcopy(nora.state_dict()))  # its own is fine


def test_train_config_records_the_optimizer_name_and_hyperparameters():
    from functools import partial

    from astrai_b200.config import TrainConfig
    from astrai_b200.optim import OptimizerFactory

    from helpers import RandomTokens

    cfg = TrainConfig(model_fn=_model, strategy="seq", dataset=RandomTokens(), optimizer_fn=partial(OptimizerFactory.create, "nora_nadamw", lr=2e-4),
                      optimizer_name="nora_nadamw", optimizer_hyperparameters={"lr": 2e-4, "nora_lr": 5e-3})
    d = cfg.to_dict()
    assert d["optimizer_name"] == "nora_nadamw" and d["optimizer_hyperparameters"] == {"lr": 2e-4, "nora_lr": 5e-3}
    assert "model_fn" not in d and "optimizer_fn" not in d  # callables never reach meta.json


def test_composite_helpers_under_the_references_names():
    from astrai_b200.optim import composite_state_dict, composite_step, composite_zero_grad, refresh_param_groups

    a, b = torch.nn.Parameter(torch.ones(2)), torch.nn.Parameter(torch.ones(3))
    first, second = torch.optim.SGD([a], lr=0.5), torch.optim.SGD([b], lr=0.25)
    ran = []

    def closure():
        ran.append(torch.is_grad_enabled())
        loss = a.sum() + b.sum()
        loss.backward()
        return loss

    with torch.no_grad():
        loss = composite_step([first, None, second], closure)
    assert ran == [True] and float(loss) == 5.0  # once, with gradients on
    assert torch.allclose(a, torch.full((2,), 0.5)) and torch.allclose(b, torch.full((3,), 0.75))
    assert [g["lr"] for g in refresh_param_groups([first, None, second])] == [0.5, 0.25]
    state = composite_state_dict({"m": first, "none": None, "rest": second})
    assert state["none"] is None and set(state["m"]) == {"state", "param_groups"}
    composite_zero_grad([first, None, second])
    assert a.grad is None and b.grad is None
    composite_zero_grad([first, second], set_to_none=False)
