"""Fused FSDP kernels (reduce-scatter + norm, AdamW + all-gather) against plain PyTorch fp32 math.

Several ranks are emulated on ONE GPU as slices of a :class:`LocalArena`.  Kernels of different ranks never wait for
one another here: all "ready" flags are preset before the launches, so every wait returns at its first poll and
the ranks' kernels simply run one after the other.  The bounded-wait test polls a flag that nothing sets, with a
0.2 s budget, and checks the status word - the GPU context stays usable.
"""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _setup(world, n_shard, seed=0):
    from astrai_b200.ops import native
    from astrai_b200.parallel.symm import LocalArena

    native.require()
    dev = torch.device("cuda")
    n = world * n_shard
    arena = LocalArena(n * 6 + (1 << 20), world, dev)
    g = torch.Generator(device="cuda").manual_seed(seed)
    ranks = []
    for r in range(world):
        a = arena.view(r)
        grad, param, flags = a.alloc(n, torch.float32), a.alloc(n, torch.bfloat16), a.alloc_flags(16)
        grad.tensor.copy_(torch.randn(n, device=dev, generator=g) * 0.1)
        ranks.append((grad, param, flags))
    w0 = (torch.randn(n, device=dev, generator=g) * 0.05).bfloat16()
    for _, param, _ in ranks:
        param.tensor.copy_(w0)
    return dev, ranks, w0


@pytest.mark.parametrize("world,n_shard", [(2, 4096), (4, 128 * 37), (8, 1024)])
def test_reduce_scatter_and_adamw_allgather_match_torch(world, n_shard):
    dev, ranks, w0 = _setup(world, n_shard)
    ops = torch.ops.astrai_b200
    unit, max_units = 3, 16
    for _, _, flags in ranks:  # every peer already "announced" epoch 1 of both kinds
        flags.tensor.fill_(1)
    full_grad = torch.stack([g.tensor for g, _, _ in ranks]).sum(0)
    lr, b1, b2, eps, wd = 1e-2, 0.9, 0.95, 1e-8, 0.1
    scale = torch.tensor([0.25], device=dev)
    total_sumsq = torch.zeros(1, device=dev)
    shards = []
    for r, (grad, param, flags) in enumerate(ranks):
        out = torch.empty(n_shard, device=dev)
        sumsq = torch.zeros(1, device=dev)
        ops.fsdp_reduce_scatter_(grad.peer_ptrs, 0, flags.peer_ptrs, r, r * n_shard, out, sumsq, unit, max_units, 1, 0.2, 8)
        ref = full_grad[r * n_shard:(r + 1) * n_shard]
        assert torch.allclose(out, ref, atol=1e-5, rtol=1e-5)
        total_sumsq += sumsq
        shards.append(out)
    assert total_sumsq.item() == pytest.approx(full_grad.pow(2).sum().item(), rel=1e-4)

    expect = torch.empty_like(w0)
    for r, (grad, param, flags) in enumerate(ranks):
        master = w0[r * n_shard:(r + 1) * n_shard].float().clone()
        m, v = torch.zeros(n_shard, device=dev), torch.zeros(n_shard, device=dev)
        counter = torch.zeros(1, dtype=torch.int32, device=dev)
        ops.fsdp_adamw_allgather_(param.peer_ptrs, 0, flags.peer_ptrs, r, r * n_shard, master, shards[r], m, v, lr, b1, b2,
                                  eps, wd, 1, scale, unit, max_units, 2, counter, 8)
        gr = shards[r] * scale
        m_ref, v_ref = (1 - b1) * gr, (1 - b2) * gr * gr
        w_ref = w0[r * n_shard:(r + 1) * n_shard].float() * (1 - lr * wd) - (lr / (1 - b1)) * m_ref / (v_ref.sqrt() / (1 - b2) ** 0.5 + eps)
        assert torch.allclose(master, w_ref, atol=1e-6, rtol=1e-5)
        assert torch.allclose(m, m_ref, atol=1e-7) and torch.allclose(v, v_ref, atol=1e-9)
        assert counter.item() == 0  # self-resetting
        expect[r * n_shard:(r + 1) * n_shard] = master.bfloat16()  # the stored parameter is the rounded master weight
    for r, (_, param, flags) in enumerate(ranks):  # every rank's full parameter buffer was written by all owners
        assert torch.equal(param.tensor, expect), r
        written = flags.tensor.view(-1, 8, max_units)[1, :world, unit]
        assert (written == 2).all()
    from astrai_b200.ops import native

    assert native.kernel_status(dev) == 0


def test_bounded_wait_reports_instead_of_hanging():
    from astrai_b200.ops import native

    dev, ranks, _ = _setup(2, 1024)
    ops = torch.ops.astrai_b200
    grad, _, flags = ranks[0]
    out, sumsq = torch.full((1024,), 7.0, device=dev), torch.zeros(1, device=dev)
    ops.kernel_status_reset(out)
    # rank 1 never announces epoch 5: the kernel gives up after 0.2 s, records the code and leaves `out` untouched
    ops.fsdp_reduce_scatter_(grad.peer_ptrs, 0, flags.peer_ptrs, 0, 0, out, sumsq, 0, 16, 5, 0.2, 4)
    assert native.kernel_status(dev) == 21
    assert (out == 7.0).all() and sumsq.item() == 0.0
    ops.kernel_status_reset(out)
    ops.comm_wait_flags_(flags.tensor, 1, 2, 0, 2, 16, 9, 0.2)
    assert native.kernel_status(dev) == 23
    ops.kernel_status_reset(out)
    assert native.kernel_status(dev) == 0
    assert torch.ones(4, device=dev).sum().item() == 4.0  # the context is still healthy
