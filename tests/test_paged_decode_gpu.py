"""Paged decode attention with the step's K / V append fused into the attention launch."""

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("hd,hq,hkv,lens", [(128, 16, 4, [513, 1, 77, 1200]), (64, 8, 8, [16, 17]), (128, 8, 1, [300])])
def test_fused_append_equals_append_then_decode(hd, hq, hkv, lens):
    op = torch.ops.astrai_b200
    g = torch.Generator(device="cuda").manual_seed(hd + hq)
    b, page, max_ctx, n_slots = len(lens), 16, 1280, 8192
    k_pool = torch.randn(n_slots, hkv, hd, device="cuda", dtype=torch.bfloat16, generator=g)
    v_pool = torch.randn(n_slots, hkv, hd, device="cuda", dtype=torch.bfloat16, generator=g)
    table = torch.zeros(b + 2, max_ctx, dtype=torch.int32, device="cuda")
    perm = torch.randperm(n_slots // page, device="cuda", generator=g)
    rows = torch.arange(b, dtype=torch.int32, device="cuda") + 1
    used = 0
    for r, n in zip(rows.tolist(), lens):
        pages = perm[used:used + -(-n // page)]
        used += pages.numel()
        table[r, :pages.numel() * page] = (pages[:, None] * page + torch.arange(page, device="cuda")[None]).reshape(-1).int()
    seq = torch.tensor(lens, dtype=torch.long, device="cuda")  # lengths include the token of this step
    q = torch.randn(b, hq, hd, device="cuda", dtype=torch.bfloat16, generator=g)
    k_new = torch.randn(b, hkv, hd, device="cuda", dtype=torch.bfloat16, generator=g)
    v_new = torch.randn(b, hkv, hd, device="cuda", dtype=torch.bfloat16, generator=g)
    splits = int(op.paged_decode_splits(b, hkv, max(lens), 8))

    def scratch():
        return (torch.zeros(b, hq, 8, hd, device="cuda"), torch.zeros(b, hq, 8, 2, device="cuda"),
                torch.zeros(b * hkv, dtype=torch.int32, device="cuda"), torch.empty_like(q))

    # two launches: append, then attend
    k1, v1 = k_pool.clone(), v_pool.clone()
    loc = torch.stack([table[r, n - 1] for r, n in zip(rows.tolist(), lens)]).int()
    op.kv_append_(k_new, v_new, k1, v1, loc)
    o_part, ml, cnt, want = scratch()
    op.paged_decode_(q, k1, v1, table, rows, seq, hd ** -0.5, splits, o_part, ml, cnt, want)
    # one launch
    k2, v2 = k_pool.clone(), v_pool.clone()
    o_part, ml, cnt, got = scratch()
    for _ in range(2):  # twice: the counters reset themselves and the stored row is idempotent
        op.paged_decode_append_(q, k_new, v_new, k2, v2, table, rows, seq, hd ** -0.5, splits, o_part, ml, cnt, got)
    torch.cuda.synchronize()
    assert torch.equal(k1, k2) and torch.equal(v1, v2)  # the pool holds the new rows, nothing else changed
    assert torch.equal(got, want)
    # fp32 statement for one request
    i = 0
    slots = table[int(rows[i]), :lens[i]].long()
    kk = k1[slots].float().repeat_interleave(hq // hkv, dim=1)
    vv = v1[slots].float().repeat_interleave(hq // hkv, dim=1)
    p = torch.softmax(torch.einsum("hd,nhd->hn", q[i].float(), kk) * hd ** -0.5, dim=-1)
    assert (got[i].float() - torch.einsum("hn,nhd->hd", p, vv)).abs().max().item() < 2e-2
