"""MoE kernels (router, plan / permute / combine, grouped GEMM forward + both gradients) against PyTorch fp32 math."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ops():
    from astrai_b200.ops import native

    native.require()
    return torch.ops.astrai_b200


@pytest.mark.parametrize("t,e,k,renorm", [(300, 64, 6, True), (1000, 8, 2, False), (77, 160, 8, True)])
def test_router_matches_torch(t, e, k, renorm):
    op = _ops()
    torch.manual_seed(0)
    logits = (torch.randn(t, e, device="cuda") * 2).bfloat16()
    probs, idx, w, counts, psum = op.moe_router(logits, k, renorm)
    ref_p = torch.softmax(logits.float(), -1).to(torch.bfloat16)
    assert (probs.float() - ref_p.float()).abs().max().item() < 1e-2
    ref_w, ref_i = torch.topk(probs.float(), k, dim=-1)
    assert torch.equal(idx.sort(-1).values, ref_i.sort(-1).values) or (probs.float().gather(1, idx).sort(-1).values - ref_w.sort(-1).values).abs().max() < 1e-6
    if renorm:
        ref_w = ref_w / ref_w.sum(-1, keepdim=True)
    assert (w.float().sort(-1).values - ref_w.sort(-1).values).abs().max().item() < 1e-2
    assert torch.equal(counts.long(), torch.bincount(idx.reshape(-1), minlength=e))
    assert torch.allclose(psum, probs.float().sum(0), rtol=1e-3, atol=1e-3)


def test_dispatch_grouped_gemm_combine_forward_and_backward():
    from astrai_b200.ops import moe, native

    op = _ops()
    torch.manual_seed(1)
    t, d, f, e, k = 520, 256, 192, 8, 2
    x = torch.randn(t, d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w1 = (torch.randn(e, f, d, device="cuda") * 0.05).bfloat16().requires_grad_(True)
    w2 = (torch.randn(e, d, f, device="cuda") * 0.05).bfloat16().requires_grad_(True)
    logits = torch.randn(t, e, device="cuda").bfloat16().requires_grad_(True)
    probs, idx, wts, counts, psum = moe.route(logits, k, True)
    xs, plan = moe.dispatch(x, idx, counts, e)
    off = plan.offsets.tolist()
    assert all(o % 128 == 0 for o in off) and [b - a for a, b in zip(off[:-1], off[1:])] == [(-(-c // 128)) * 128 for c in counts.tolist()]
    te = plan.tile_expert.tolist()
    for ei in range(e):
        assert all(te[j] == ei for j in range(off[ei] // 128, off[ei + 1] // 128))
    assert all(v == -1 for v in te[off[-1] // 128:])
    # every (token, choice) row sits inside its expert's segment and holds the token's activations
    slot = plan.slot_of
    assert torch.equal(xs[slot.reshape(-1).long()], x.detach()[torch.arange(t, device="cuda").repeat_interleave(k)])
    seg = torch.tensor(off, device="cuda")
    assert ((slot >= seg[idx]) & (slot < seg[idx + 1])).all()
    h = moe.zero_unused_rows(moe.grouped_linear(xs, w1, plan), plan)
    y = moe.zero_unused_rows(moe.grouped_linear(torch.nn.functional.silu(h.float()).to(h.dtype), w2, plan), plan)
    out = moe.combine(y, wts, plan)
    # reference: per-token dense evaluation in fp32
    xf, w1f, w2f = x.detach().float().requires_grad_(True), w1.detach().float().requires_grad_(True), w2.detach().float().requires_grad_(True)
    wtf = wts.detach().float().requires_grad_(True)
    hh = torch.einsum("td,tkfd->tkf", xf, w1f[idx])
    yy = torch.einsum("tkf,tkdf->tkd", torch.nn.functional.silu(hh), w2f[idx])
    ref = (yy * wtf[..., None]).sum(1)
    assert (out.float() - ref).abs().max().item() < 3e-2 * ref.abs().max().item() + 1e-2
    g = torch.randn_like(out)
    out.backward(g)
    ref.backward(g.float())
    for name, a, b in (("dx", x.grad, xf.grad), ("dw1", w1.grad, w1f.grad), ("dw2", w2.grad, w2f.grad)):
        assert (a.float() - b).abs().max().item() < 4e-2 * b.abs().max().item() + 1e-3, name
    assert logits.grad is not None and torch.isfinite(logits.grad.float()).all()
    assert native.kernel_status(x.device) == 0


def test_moe_module_kernel_path_matches_torch_path():
    from astrai_b200.models.ffn import DeepSeekMoE

    torch.manual_seed(2)
    moe_mod = DeepSeekMoE(dim=256, dim_ffn=512, n_routed_experts=8, n_shared_experts=1, n_activated_experts=2, moe_intermediate_size=192).to("cuda", torch.bfloat16)
    with torch.no_grad():
        for p in moe_mod.parameters():
            p.normal_(std=0.05)
    x = torch.randn(4, 96, 256, device="cuda", dtype=torch.bfloat16)
    moe_mod.train()
    out_k = moe_mod(x)
    moe_mod.expert_parallel = None
    ref_w, ref_i, aux, _ = moe_mod.route(x.reshape(-1, 256), True)
    out_t = moe_mod._routed(x.reshape(-1, 256), ref_w, ref_i)
    shared = moe_mod.shared_experts[0](x.reshape(-1, 256))["hidden_states"]
    ref = (out_t + shared).view_as(x)
    assert (out_k["hidden_states"].float() - ref.float()).abs().max().item() < 5e-2 * ref.float().abs().max().item() + 2e-2
    assert abs(out_k["aux_loss"].item() - aux.item()) < 2e-2 * abs(aux.item()) + 1e-3
