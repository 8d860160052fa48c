"""Zig-zag sequence sharding helpers of context-parallel attention (CPU)."""

import pytest
import torch

from astrai_b200.parallel import context_parallel as cpar


@pytest.mark.parametrize("world", [2, 3, 4])
def test_zigzag_roundtrip_and_positions(world):
    s = 2 * world * 3
    x = torch.arange(2 * s * 5).view(2, s, 5)
    parts = [cpar.zigzag_split(x, world, r) for r in range(world)]
    assert all(p.shape == (2, s // world, 5) for p in parts)
    assert torch.equal(cpar.zigzag_merge(parts), x)
    for r in range(world):
        pos = cpar.zigzag_positions(s, world, r)
        assert torch.equal(x[:, pos], parts[r])
    # every rank sees the same number of (query, key) pairs under a causal mask
    work = [int((cpar.zigzag_positions(s, world, r) + 1).sum()) for r in range(world)]
    assert len(set(work)) == 1


def test_zigzag_split_rejects_ragged_length():
    with pytest.raises(ValueError):
        cpar.zigzag_split(torch.zeros(1, 10, 2), 2, 0)


def test_reference_matches_unsharded_attention():
    torch.manual_seed(0)
    world, s = 2, 16
    q, k, v = torch.randn(1, s, 4, 8), torch.randn(1, s, 2, 8), torch.randn(1, s, 2, 8)
    outs = cpar.ring_attention_reference([cpar.zigzag_split(q, world, r) for r in range(world)],
                                         [cpar.zigzag_split(k, world, r) for r in range(world)],
                                         [cpar.zigzag_split(v, world, r) for r in range(world)])
    kk, vv = k.repeat_interleave(2, dim=2), v.repeat_interleave(2, dim=2)
    full = torch.nn.functional.scaled_dot_product_attention(q.transpose(1, 2), kk.transpose(1, 2), vv.transpose(1, 2),
                                                            is_causal=True).transpose(1, 2)
    assert torch.allclose(cpar.zigzag_merge(outs), full, atol=1e-6)


def test_ring_attention_needs_context():
    cpar.set_context(None)
    with pytest.raises(RuntimeError):
        cpar.ring_attention(torch.zeros(1, 256, 2, 64), torch.zeros(1, 256, 2, 64), torch.zeros(1, 256, 2, 64))
