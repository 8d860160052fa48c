"""Expert-parallel MoE (routing exchange, grouped GEMM with gather / scatter over peer memory) against fp32 PyTorch.

Ranks are emulated on one GPU as slices of a :class:`LocalArena`; the pass runs phase by phase - phase i of every rank
before phase i + 1 of any - so no kernel ever waits for a kernel that has not run yet.  The one flag that a kernel
both publishes and waits for in the same launch (the gradient announcement) is preset.
"""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _make(world, t, h, f, e, k, seed=2):
    from astrai_b200.ops import native
    from astrai_b200.parallel import expert_parallel as epar
    from astrai_b200.parallel.symm import LocalArena

    native.require()
    g = torch.Generator(device="cuda").manual_seed(seed)
    xs = [torch.randn(t, h, device="cuda", generator=g).bfloat16() for _ in range(world)]
    router = (torch.randn(e, h, device="cuda", generator=g) * 0.1).bfloat16()
    gate_up = (torch.randn(e, 2 * f, h, device="cuda", generator=g) * 0.05).bfloat16()
    down = (torch.randn(e, h, f, device="cuda", generator=g) * 0.05).bfloat16()
    arena = LocalArena(epar.arena_bytes_for(t, h, k, world, e), world, torch.device("cuda"))
    ctxs = [epar.EPContext(arena.view(r), r, world, timeout_s=0.5, n_copy_ctas=3) for r in range(world)]
    return epar, xs, router, gate_up, down, ctxs


def _route(x, router, k):
    from astrai_b200.ops import moe

    logits = (x.float() @ router.float().t()).to(x.dtype)
    return moe.route(logits, k, True)


@pytest.mark.parametrize("world,t,h,f,e,k", [(2, 192, 128, 64, 4, 2), (4, 256, 256, 128, 8, 3)])
def test_expert_parallel_forward_backward_emulated_ranks(world, t, h, f, e, k):
    from astrai_b200.ops import native
    from astrai_b200.parallel import symm

    epar, xs, router, gate_up, down, ctxs = _make(world, t, h, f, e, k)
    el = e // world
    r_cap = epar.row_capacity(t, k, world, el)
    routed = [_route(x, router, k) for x in xs]  # probs, idx, weights, counts, psum
    sts = [epar._fwd_push(ctxs[r], xs[r], routed[r][1], routed[r][3], r_cap) for r in range(world)]
    for st in sts:
        epar._fwd_plan(st)
    w_gu = [gate_up[r * el:(r + 1) * el].contiguous() for r in range(world)]
    w_dn = [down[r * el:(r + 1) * el].contiguous() for r in range(world)]
    for r, st in enumerate(sts):
        epar._fwd_experts(st, w_gu[r], w_dn[r])
    outs = [epar._fwd_combine(st, routed[r][2]) for r, st in enumerate(sts)]
    assert native.kernel_status(torch.device("cuda")) == 0

    # the plan: every rank's segments hold exactly the pairs that chose its experts
    all_idx = torch.stack([routed[r][1] for r in range(world)])  # [W, T, K]
    for r, st in enumerate(sts):
        mine = ((all_idx // el) == r).sum().item()
        assert (st.row_peer >= 0).sum().item() == mine
        off = st.offsets.tolist()
        assert off[-1] == st.total.item() and all(o % 128 == 0 for o in off)
        for le in range(el):
            seg = st.row_peer[off[le]:off[le + 1]]
            seg = seg[seg >= 0]
            src, pair = seg >> 24, seg & 0xFFFFFF
            assert (all_idx.view(world, -1)[src.long(), pair.long()] == r * el + le).all()
            assert (src[1:] >= src[:-1]).all()  # rows of source rank 0 first, then rank 1, ...

    # fp32 reference with the SAME routing decisions
    def reference(x_list, wts):
        res = []
        for r in range(world):
            xf = x_list[r]
            out = torch.zeros(t, h, device="cuda")
            idx = routed[r][1]
            for ee in range(e):
                sel = idx == ee
                rows = sel.any(-1).nonzero().flatten()
                if rows.numel() == 0:
                    continue
                hgu = xf[rows] @ gate_up[ee].float().t()
                act = torch.nn.functional.silu(hgu[:, :f]) * hgu[:, f:]
                out[rows] += (wts[r][rows] * sel[rows]).sum(-1, keepdim=True) * (act @ down[ee].float().t())
            res.append(out)
        return res

    xr = [x.float().requires_grad_(True) for x in xs]
    wr = [routed[r][2].detach().float().requires_grad_(True) for r in range(world)]
    refs = reference(xr, wr)
    for r in range(world):
        err = (outs[r].float() - refs[r]).abs().max().item()
        assert err <= 0.03 * refs[r].abs().max().item() + 1e-3, (r, err)

    # backward
    g = torch.Generator(device="cuda").manual_seed(9)
    douts = [torch.randn(t, h, device="cuda", generator=g).bfloat16() for _ in range(world)]
    gu32, dn32 = gate_up.float().requires_grad_(True), down.float().requires_grad_(True)
    gate_up, down = gu32, dn32  # the closure above now differentiates through fp32 leaves
    refs = reference(xr, wr)
    torch.autograd.backward(refs, [d.float() for d in douts])
    dweights = [epar._bwd_prepare(st, douts[r], routed[r][2].detach()) for r, st in enumerate(sts)]
    for cx in ctxs:  # every peer has announced its gradient rows
        cx.flags.tensor.view(-1, 8, epar.MAX_UNITS)[symm.KIND_EP, :, epar.U_DY] = sts[0].be
    grads = [epar._bwd_experts(st, w_gu[r], w_dn[r]) for r, st in enumerate(sts)]
    dxs = [epar._bwd_finish(st) for st in sts]
    assert native.kernel_status(torch.device("cuda")) == 0

    def close(a, b, tol=0.04):
        return (a.float() - b).abs().max().item() <= tol * b.abs().max().item() + 1e-3

    for r in range(world):
        assert close(dxs[r], xr[r].grad), r
        assert close(dweights[r], wr[r].grad), r
        assert close(grads[r][0], gu32.grad[r * el:(r + 1) * el]), r
        assert close(grads[r][1], dn32.grad[r * el:(r + 1) * el]), r


def test_plan_reports_a_missing_peer_instead_of_hanging():
    from astrai_b200.ops import native

    epar, xs, router, gate_up, down, ctxs = _make(2, 128, 128, 64, 4, 2)
    ops = torch.ops.astrai_b200
    routed = _route(xs[0], router, 2)
    st = epar._fwd_push(ctxs[0], xs[0], routed[1], routed[3], epar.row_capacity(128, 2, 2, 2))
    ops.kernel_status_reset(xs[0])
    epar._fwd_plan(st)  # rank 1 never pushed its counts: the bounded wait runs out
    torch.cuda.synchronize()
    assert native.kernel_status(torch.device("cuda")) == 71
    ops.kernel_status_reset(xs[0])
    assert torch.zeros(4, device="cuda").sum().item() == 0
