"""Context-parallel flash attention against fp32 PyTorch attention of the whole sequence.

Ranks are emulated on one GPU: each "rank" is a slice of a :class:`LocalArena` and its kernels run one after the other.
For the fused gather every peer's "K / V ready" flag is preset, so no kernel waits for another rank's kernel; in the
backward pass all ranks scatter first and the owners reduce afterwards.
"""

import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _setup(world, c, b, hq, hkv, d, seed=3):
    from astrai_b200.ops import native
    from astrai_b200.parallel import context_parallel as cpar

    native.require()
    s = 2 * world * c
    g = torch.Generator(device="cuda").manual_seed(seed)
    q = torch.randn(b, s, hq, d, device="cuda", generator=g).bfloat16()
    k = torch.randn(b, s, hkv, d, device="cuda", generator=g).bfloat16()
    v = torch.randn(b, s, hkv, d, device="cuda", generator=g).bfloat16()
    do = torch.randn(b, s, hq, d, device="cuda", generator=g).bfloat16()
    qr, kr, vr = (t.float().requires_grad_(True) for t in (q, k, v))
    grp = hq // hkv
    ref = torch.nn.functional.scaled_dot_product_attention(
        qr.transpose(1, 2), kr.repeat_interleave(grp, dim=2).transpose(1, 2), vr.repeat_interleave(grp, dim=2).transpose(1, 2),
        is_causal=True).transpose(1, 2)
    ref.backward(do.float())
    return cpar, (q, k, v, do), (ref.detach(), qr.grad, kr.grad, vr.grad)


def _close(a, ref, tol):
    return (a.float() - ref).abs().max().item() <= tol * ref.abs().max().item() + 1e-3


@pytest.mark.parametrize("world,c,b,hq,hkv,d", [(2, 128, 1, 4, 2, 128), (4, 256, 2, 4, 4, 64), (3, 128, 1, 8, 2, 128)])
def test_sharded_kernels_on_gathered_keys(world, c, b, hq, hkv, d):
    """The zig-zag masks and the key-tile visiting order alone: K / V gathered by PyTorch, partial dK / dV summed here."""
    cpar, (q, k, v, do), (ref, dq_ref, dk_ref, dv_ref) = _setup(world, c, b, hq, hkv, d)
    ops = torch.ops.astrai_b200
    s, scale = 2 * world * c, 1.0 / math.sqrt(d)
    k_full, v_full = k.reshape(b * s, hkv, d), v.reshape(b * s, hkv, d)
    dk_sum = torch.zeros(b * s, hkv, d, device="cuda")
    dv_sum = torch.zeros_like(dk_sum)
    for r in range(world):
        ql = cpar.zigzag_split(q, world, r).reshape(b * 2 * c, hq, d)
        dol = cpar.zigzag_split(do, world, r).reshape(b * 2 * c, hq, d)
        out, lse = ops.cp_flash_fwd(ql, k_full, v_full, b, c, world, r, scale, [], [], 0, 1, 0, 0, None, 1.0)
        assert _close(out.view(b, 2 * c, hq, d), cpar.zigzag_split(ref, world, r), 0.02), r
        dq, dk, dv = ops.cp_flash_bwd(ql, k_full, v_full, out, dol, lse, b, c, world, r, scale, [], [], 0, 1, 0, None, 1.0)
        assert _close(dq.view(b, 2 * c, hq, d), cpar.zigzag_split(dq_ref, world, r), 0.03), r
        vis = (2 * world - r) * c
        if vis < s:  # nothing written for keys this rank cannot see
            assert dk.view(b, s, hkv, d)[:, vis:].abs().max().item() == 0
        dk_sum += dk.float()
        dv_sum += dv.float()
    assert _close(dk_sum.view(b, s, hkv, d), dk_ref, 0.03)
    assert _close(dv_sum.view(b, s, hkv, d), dv_ref, 0.03)
    from astrai_b200.ops import native

    assert native.kernel_status(torch.device("cuda")) == 0


@pytest.mark.parametrize("world,c,b,hq,hkv,d,n_copy", [(2, 128, 1, 4, 2, 128, 2), (4, 128, 2, 4, 2, 64, 3), (2, 384, 1, 2, 1, 128, 8)])
def test_fused_gather_and_scatter_emulated_ranks(world, c, b, hq, hkv, d, n_copy):
    from astrai_b200.ops import native
    from astrai_b200.parallel.symm import LocalArena

    cpar, (q, k, v, do), (ref, dq_ref, dk_ref, dv_ref) = _setup(world, c, b, hq, hkv, d, seed=11)
    ops = torch.ops.astrai_b200
    s, scale, row = 2 * world * c, 1.0 / math.sqrt(d), hkv * d
    arena = LocalArena(cpar.arena_bytes_for(b, s, world, hkv, d), world, torch.device("cuda"))
    ctxs = [cpar.CPContext(arena.view(r), r, world, timeout_s=0.5, n_copy_ctas=n_copy) for r in range(world)]
    srcs = [cx.kv_source(b, c, row, 1) for cx in ctxs]
    stages = [cx.stage(b, c, row, 0) for cx in ctxs]
    for r, cx in enumerate(ctxs):
        pair = srcs[r].tensor.view(2, b, 2 * c, hkv, d)
        pair[0].copy_(cpar.zigzag_split(k, world, r))
        pair[1].copy_(cpar.zigzag_split(v, world, r))
        cx.flags.tensor.view(-1, 8, 1)[4].fill_(1)  # plane "K / V ready": every peer has announced epoch 1
    saved = []
    for r, cx in enumerate(ctxs):
        ql = cpar.zigzag_split(q, world, r).reshape(b * 2 * c, hq, d)
        k_full = torch.zeros(b * s, hkv, d, device="cuda", dtype=torch.bfloat16)
        v_full = torch.zeros_like(k_full)
        out, lse = ops.cp_flash_fwd(ql, k_full, v_full, b, c, world, r, scale, srcs[r].peer_ptrs, cx.flags.peer_ptrs, 0, 1, 1,
                                    n_copy, cx.chunk_state, 0.5)
        assert torch.equal(k_full.view(b, s, hkv, d), k) and torch.equal(v_full.view(b, s, hkv, d), v), r
        assert _close(out.view(b, 2 * c, hq, d), cpar.zigzag_split(ref, world, r), 0.02), r
        assert (cx.chunk_state[:world] == 1).all() and cx.chunk_state[8:].sum().item() == 0
        saved.append((ql, k_full, v_full, out, lse))
    assert native.kernel_status(torch.device("cuda")) == 0
    for r, cx in enumerate(ctxs):  # every rank scatters its partial dK / dV tiles to the owners' staging slots
        ql, k_full, v_full, out, lse = saved[r]
        dol = cpar.zigzag_split(do, world, r).reshape(b * 2 * c, hq, d)
        dq, _, _ = ops.cp_flash_bwd(ql, k_full, v_full, out, dol, lse, b, c, world, r, scale, stages[r].peer_ptrs,
                                    cx.flags.peer_ptrs, 0, 1, 2, cx.tile_counter, 0.5)
        assert _close(dq.view(b, 2 * c, hq, d), cpar.zigzag_split(dq_ref, world, r), 0.03), r
        assert cx.tile_counter.sum().item() == 0
    for r, cx in enumerate(ctxs):  # the owners sum what has arrived
        got = cx.flags.tensor.view(-1, 8, 1)[6, :world, 0]
        assert (got == 2).all(), (r, got)  # every source published "my tiles for rank r are written" with the epoch
        dk = torch.empty(b * 2 * c, hkv, d, device="cuda", dtype=torch.bfloat16)
        dv = torch.empty_like(dk)
        ops.cp_dkv_reduce(dk, dv, b, c, world, r, stages[r].peer_ptrs, cx.flags.peer_ptrs, 0, 1, 2, 0.5)
        assert _close(dk.view(b, 2 * c, hkv, d), cpar.zigzag_split(dk_ref, world, r), 0.03), r
        assert _close(dv.view(b, 2 * c, hkv, d), cpar.zigzag_split(dv_ref, world, r), 0.03), r
    assert native.kernel_status(torch.device("cuda")) == 0


def test_reduce_reports_a_missing_peer_instead_of_hanging():
    """A flag that nothing sets: the bounded wait runs out, the status word carries the code, the context stays usable."""
    from astrai_b200.ops import native
    from astrai_b200.parallel.symm import LocalArena

    cpar, _, _ = _setup(2, 128, 1, 2, 1, 64)
    ops = torch.ops.astrai_b200
    arena = LocalArena(cpar.arena_bytes_for(1, 512, 2, 1, 64), 2, torch.device("cuda"))
    cx = cpar.CPContext(arena.view(0), 0, 2, timeout_s=0.2)
    stage = cx.stage(1, 128, 64, 0)
    dk = torch.zeros(256, 1, 64, device="cuda", dtype=torch.bfloat16)
    dv = torch.zeros_like(dk)
    ops.kernel_status_reset(dk)
    ops.cp_dkv_reduce(dk, dv, 1, 128, 2, 0, stage.peer_ptrs, cx.flags.peer_ptrs, 0, 1, 5, 0.2)
    torch.cuda.synchronize()
    assert native.kernel_status(torch.device("cuda")) == 63
    ops.kernel_status_reset(dk)
    assert torch.zeros(4, device="cuda").sum().item() == 0  # the context still works
