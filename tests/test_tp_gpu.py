"""Fused tensor-parallel GEMMs (all-gather -> GEMM, GEMM -> reduce-scatter) against fp32 PyTorch math.

Ranks are emulated on one GPU as slices of a :class:`LocalArena`; every "ready" flag is preset, so no kernel waits
for another rank's kernel, and the reduce phase of the reduce-scatter runs as a separate launch after all ranks
have scattered their tiles.
"""

import pytest
import torch

pytestmark = pytest.mark.gpu

MAX_UNITS = 64


def _arena(world, nbytes):
    from astrai_b200.ops import native
    from astrai_b200.parallel.symm import LocalArena

    native.require()
    return LocalArena(nbytes, world, torch.device("cuda"))


@pytest.mark.parametrize("world,ms,k,n,w_kmajor", [(2, 128, 256, 512, True), (4, 256, 320, 288, True), (2, 128, 192, 256, False)])
def test_allgather_gemm_matches_torch(world, ms, k, n, w_kmajor):
    ops = torch.ops.astrai_b200
    m = world * ms
    arena = _arena(world, m * k * 2 + (1 << 20))
    g = torch.Generator(device="cuda").manual_seed(5)
    xs = [torch.randn(ms, k, device="cuda", generator=g).bfloat16() for _ in range(world)]
    ws = [(torch.randn(n, k, device="cuda", generator=g) * 0.05).bfloat16() for _ in range(world)]
    bufs, flags = [], []
    for r in range(world):
        a = arena.view(r)
        bufs.append(a.alloc(m * k, torch.bfloat16))
        flags.append(a.alloc_flags(MAX_UNITS))
        bufs[r].tensor.view(m, k)[r * ms:(r + 1) * ms].copy_(xs[r])
        flags[r].tensor.fill_(1)  # every peer has announced epoch 1
    x_full = torch.cat(xs).float()
    for r in range(world):
        w = ws[r] if w_kmajor else ws[r].t().contiguous()
        y = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)
        cf, cc = torch.zeros(8, dtype=torch.int32, device="cuda"), torch.zeros(8, dtype=torch.int32, device="cuda")
        ops.tp_gemm_allgather_(bufs[r].peer_ptrs, w, w_kmajor, y, flags[r].peer_ptrs, cf, cc, r, 0, MAX_UNITS, 1, 0.5, 4)
        ref = x_full @ ws[r].float().t()
        assert torch.equal(bufs[r].tensor.view(m, k).float(), x_full), r  # the gathered activations are exact copies
        assert (y.float() - ref).abs().max().item() < 0.05 * ref.abs().max().item() + 1e-2, r
        assert cc.sum().item() == 0 and (cf[[i for i in range(world) if i != r]] == 1).all()
    from astrai_b200.ops import native

    assert native.kernel_status(torch.device("cuda")) == 0


@pytest.mark.parametrize("world,ms,kp,n,w_kmajor", [(2, 128, 256, 512, True), (4, 128, 192, 320, True), (2, 256, 128, 256, False)])
def test_gemm_reducescatter_matches_torch(world, ms, kp, n, w_kmajor):
    ops = torch.ops.astrai_b200
    m = world * ms
    arena = _arena(world, world * ms * n * 2 + (1 << 20))
    g = torch.Generator(device="cuda").manual_seed(6)
    xs = [torch.randn(m, kp, device="cuda", generator=g).bfloat16() for _ in range(world)]
    ws = [(torch.randn(n, kp, device="cuda", generator=g) * 0.05).bfloat16() for _ in range(world)]
    stages, flags = [], []
    for r in range(world):
        a = arena.view(r)
        stages.append(a.alloc(world * ms * n, torch.bfloat16))
        flags.append(a.alloc_flags(MAX_UNITS))
    outs = [torch.empty(ms, n, device="cuda", dtype=torch.bfloat16) for _ in range(world)]
    for r in range(world):
        w = ws[r] if w_kmajor else ws[r].t().contiguous()
        tc = torch.zeros(8, dtype=torch.int32, device="cuda")
        ops.tp_gemm_reducescatter_(xs[r], w, w_kmajor, stages[r].peer_ptrs, outs[r], flags[r].peer_ptrs, tc, r, 1, MAX_UNITS, 3,
                                   0.5, False)
    full = sum(x.float() @ w.float().t() for x, w in zip(xs, ws))
    for r in range(world):
        ops.tp_reduce_(stages[r].tensor, outs[r], world)
        ref = full[r * ms:(r + 1) * ms]
        assert (outs[r].float() - ref).abs().max().item() < 0.03 * ref.abs().max().item() + 1e-2, r
        # every source published "all tiles for rank r are written" (plane 3, slot 1) with the epoch
        got = flags[r].tensor.view(-1, 8, MAX_UNITS)[3, :world, 1]
        assert (got == 3).all(), r
    from astrai_b200.ops import native

    assert native.kernel_status(torch.device("cuda")) == 0


@pytest.mark.parametrize("world,ms,k,n,w_kmajor", [(2, 256, 256, 512, True), (4, 512, 320, 288, True), (2, 256, 192, 256, False),
                                                   (8, 256, 128, 96, True)])
@pytest.mark.parametrize("slots", [1, 2, 3])
def test_pair_engine_allgather_gemm_matches_torch(world, ms, k, n, w_kmajor, slots):
    """The CTA-pair kernel whose extra warp pulls the peers' row blocks with bulk copies (ranks emulated on one GPU,
    announcements preset so that no kernel waits for another).  ``slots``: copy slots of the comm lane, each taken from
    the GEMM's operand stages (6 + 1, 5 + 2, 4 + 3)."""
    ops = torch.ops.astrai_b200
    m = world * ms
    arena = _arena(world, m * k * 2 + (1 << 20))
    g = torch.Generator(device="cuda").manual_seed(15)
    xs = [torch.randn(ms, k, device="cuda", generator=g).bfloat16() for _ in range(world)]
    ws = [(torch.randn(n, k, device="cuda", generator=g) * 0.05).bfloat16() for _ in range(world)]
    bufs, flags = [], []
    for r in range(world):
        a = arena.view(r)
        bufs.append(a.alloc(m * k, torch.bfloat16))
        flags.append(a.alloc_flags(MAX_UNITS))
        bufs[r].tensor.view(m, k)[r * ms:(r + 1) * ms].copy_(xs[r])
        flags[r].tensor.fill_(1)
    x_full = torch.cat(xs).float()
    for r in range(world):
        w = ws[r] if w_kmajor else ws[r].t().contiguous()
        y = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)
        cf, cc = torch.zeros(8, dtype=torch.int32, device="cuda"), torch.zeros(8, dtype=torch.int32, device="cuda")
        for epoch in (1, 1):  # twice: counters reset themselves, flags stay at the epoch
            ops.tp2_gemm_allgather_(bufs[r].peer_ptrs, w, w_kmajor, y, flags[r].peer_ptrs, cf, cc, r, 0, MAX_UNITS, epoch, 0.5, slots)
        ref = x_full @ ws[r].float().t()
        assert torch.equal(bufs[r].tensor.view(m, k).float(), x_full), r
        assert (y.float() - ref).abs().max().item() < 0.05 * ref.abs().max().item() + 1e-2, r
        assert cc.sum().item() == 0 and (cf[[i for i in range(world) if i != r]] == 1).all()
    from astrai_b200.ops import native

    assert native.kernel_status(torch.device("cuda")) == 0


@pytest.mark.parametrize("world,ms,kp,n,w_kmajor", [(2, 256, 256, 512, True), (4, 256, 192, 320, True), (2, 512, 128, 256, False),
                                                    (8, 256, 64, 128, True)])
@pytest.mark.parametrize("slots", [1, 2, 3])
def test_pair_engine_gemm_reducescatter_matches_torch(world, ms, kp, n, w_kmajor, slots):
    """Reduce-scatter by pulling: phase 0 of every rank (partial product + announcements), then phase 2 of every rank
    (pull the peers' blocks with bulk copies, sum in fp32), so that no kernel waits for another one on this one GPU."""
    ops = torch.ops.astrai_b200
    m = world * ms
    arena = _arena(world, m * n * 2 + (1 << 20))
    g = torch.Generator(device="cuda").manual_seed(16)
    xs = [torch.randn(m, kp, device="cuda", generator=g).bfloat16() for _ in range(world)]
    ws = [(torch.randn(n, kp, device="cuda", generator=g) * 0.05).bfloat16() for _ in range(world)]
    parts, flags = [], []
    for r in range(world):
        a = arena.view(r)
        parts.append(a.alloc(m * n, torch.bfloat16))
        flags.append(a.alloc_flags(MAX_UNITS))
    outs = [torch.full((ms, n), float("nan"), device="cuda", dtype=torch.bfloat16) for _ in range(world)]
    gath = [torch.zeros(world * ms * n, device="cuda", dtype=torch.bfloat16) for _ in range(world)]
    tcs = [torch.zeros(8, dtype=torch.int32, device="cuda") for _ in range(world)]
    pcs = [torch.zeros(1, dtype=torch.int32, device="cuda") for _ in range(world)]
    for phase in (0, 2):
        for r in range(world):
            w = ws[r] if w_kmajor else ws[r].t().contiguous()
            ops.tp2_gemm_reducescatter_(xs[r], w, w_kmajor, parts[r].peer_ptrs, gath[r], outs[r], flags[r].peer_ptrs, tcs[r], pcs[r],
                                        r, 1, MAX_UNITS, 3, 0.5, phase, slots)
    full = sum(x.float() @ w.float().t() for x, w in zip(xs, ws))
    for r in range(world):
        ref = full[r * ms:(r + 1) * ms]
        assert (outs[r].float() - ref).abs().max().item() < 0.03 * ref.abs().max().item() + 1e-2, r
        got = flags[r].tensor.view(-1, 8, MAX_UNITS)[3, :world, 1]
        assert (got == 3).all(), r
        mine = parts[r].tensor.view(m, n).float()  # the whole partial product of rank r sits in its symmetric buffer
        want = xs[r].float() @ ws[r].float().t()
        assert (mine - want).abs().max().item() < 0.03 * want.abs().max().item() + 1e-2
    from astrai_b200.ops import native

    assert native.kernel_status(torch.device("cuda")) == 0
