"""tcgen05 flash attention (forward and backward) against a plain fp32 PyTorch statement of the same math."""

import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref_attention(q, k, v, causal, scale):
    """q [Sq,Hq,D], k/v [Sk,Hkv,D] fp32; lower-right aligned causal mask.  Returns (out [Sq,Hq,D], lse [Hq,Sq])."""
    sq, hq, _ = q.shape
    sk, hkv, _ = k.shape
    kk = k.repeat_interleave(hq // hkv, dim=1)
    vv = v.repeat_interleave(hq // hkv, dim=1)
    s = torch.einsum("qhd,khd->hqk", q, kk) * scale
    if causal:
        i = torch.arange(sq, device=q.device)[:, None]
        j = torch.arange(sk, device=q.device)[None, :]
        s = s.masked_fill(~(j <= i + (sk - sq)), float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    p = torch.softmax(s, dim=-1)
    p = torch.nan_to_num(p, nan=0.0)
    return torch.einsum("hqk,khd->qhd", p, vv), lse


def _native():
    from astrai_b200.ops import native

    native.require()
    return torch.ops.astrai_b200


@pytest.mark.parametrize("d", [128, 64])
@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("b,s,hq,hkv", [(2, 256, 4, 2), (1, 384, 2, 2), (3, 200, 4, 1)])
def test_flash_fwd_dense(d, causal, b, s, hq, hkv):
    ops = _native()
    torch.manual_seed(0)
    q = torch.randn(b * s, hq, d, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(b * s, hkv, d, device="cuda", dtype=torch.bfloat16)
    v = torch.randn(b * s, hkv, d, device="cuda", dtype=torch.bfloat16)
    scale = 1.0 / math.sqrt(d)
    out, lse = ops.flash_fwd(q, k, v, None, None, b, s, s, s, causal, scale)
    for i in range(b):
        sl = slice(i * s, (i + 1) * s)
        ref, ref_lse = _ref_attention(q[sl].float(), k[sl].float(), v[sl].float(), causal, scale)
        assert (out[sl].float() - ref).abs().max().item() < 2e-2
        assert (lse[:, sl] - ref_lse).abs().max().item() < 2e-2
    from astrai_b200.ops import native

    assert native.kernel_status(q.device) == 0


@pytest.mark.parametrize("d", [128, 64])
def test_flash_fwd_varlen_with_prefix(d):
    ops = _native()
    torch.manual_seed(1)
    hq, hkv = 4, 2
    q_lens, k_lens = [130, 1, 77, 256], [130, 300, 200, 256]  # k_len >= q_len: queries sit at the end of their keys
    cu_q = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32, device="cuda")
    cu_k = torch.tensor([0] + list(torch.tensor(k_lens).cumsum(0)), dtype=torch.int32, device="cuda")
    q = torch.randn(sum(q_lens), hq, d, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(sum(k_lens), hkv, d, device="cuda", dtype=torch.bfloat16)
    v = torch.randn(sum(k_lens), hkv, d, device="cuda", dtype=torch.bfloat16)
    scale = 1.0 / math.sqrt(d)
    out, lse = ops.flash_fwd(q, k, v, cu_q, cu_k, len(q_lens), 0, 0, max(q_lens), True, scale)
    for i in range(len(q_lens)):
        qs = slice(int(cu_q[i]), int(cu_q[i + 1]))
        ks = slice(int(cu_k[i]), int(cu_k[i + 1]))
        ref, ref_lse = _ref_attention(q[qs].float(), k[ks].float(), v[ks].float(), True, scale)
        assert (out[qs].float() - ref).abs().max().item() < 2e-2, i
        assert (lse[:, qs] - ref_lse).abs().max().item() < 2e-2, i


def _ref_grads(q, k, v, do, causal, scale):
    q, k, v = (t.float().detach().requires_grad_(True) for t in (q, k, v))
    out, _ = _ref_attention(q, k, v, causal, scale)
    out.backward(do.float())
    return q.grad, k.grad, v.grad


def _close(a, b, tol):
    denom = b.abs().max().item() + 1e-6
    return (a.float() - b).abs().max().item() / denom < tol


@pytest.mark.parametrize("d", [128, 64])
@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("b,s,hq,hkv", [(2, 256, 4, 2), (1, 320, 2, 2), (2, 200, 4, 1)])
def test_flash_bwd_dense(d, causal, b, s, hq, hkv):
    ops = _native()
    torch.manual_seed(2)
    q = torch.randn(b * s, hq, d, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(b * s, hkv, d, device="cuda", dtype=torch.bfloat16)
    v = torch.randn(b * s, hkv, d, device="cuda", dtype=torch.bfloat16)
    do = torch.randn(b * s, hq, d, device="cuda", dtype=torch.bfloat16)
    scale = 1.0 / math.sqrt(d)
    out, lse = ops.flash_fwd(q, k, v, None, None, b, s, s, s, causal, scale)
    dq, dk, dv = ops.flash_bwd(q, k, v, out, do, lse, None, None, b, s, s, s, s, causal, scale)
    for i in range(b):
        sl = slice(i * s, (i + 1) * s)
        rq, rk, rv = _ref_grads(q[sl], k[sl], v[sl], do[sl], causal, scale)
        assert _close(dv[sl], rv, 2e-2), ("dv", i)
        assert _close(dk[sl], rk, 2e-2), ("dk", i)
        assert _close(dq[sl], rq, 2e-2), ("dq", i)
    from astrai_b200.ops import native

    assert native.kernel_status(q.device) == 0


@pytest.mark.parametrize("b,s,hq,hkv,d", [(4, 2048, 16, 4, 128), (3, 1152, 8, 2, 64)])
def test_flash_many_items_per_cta(b, s, hq, hkv, d):
    """More work items than resident CTAs (the persistent forward kernel walks several items per CTA, so its barrier
    phases, Q tile and O accumulator are reused) and long key / query loops in the backward kernels (every ring wraps
    many times).  Forward and backward against the fp32 statement, sequence by sequence."""
    ops = _native()
    torch.manual_seed(5)
    q = torch.randn(b * s, hq, d, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(b * s, hkv, d, device="cuda", dtype=torch.bfloat16)
    v = torch.randn(b * s, hkv, d, device="cuda", dtype=torch.bfloat16)
    do = torch.randn(b * s, hq, d, device="cuda", dtype=torch.bfloat16)
    scale = 1.0 / math.sqrt(d)
    out, lse = ops.flash_fwd(q, k, v, None, None, b, s, s, s, True, scale)
    dq, dk, dv = ops.flash_bwd(q, k, v, out, do, lse, None, None, b, s, s, s, s, True, scale)
    assert not torch.isnan(out).any() and not torch.isnan(dq).any() and not torch.isnan(dk).any() and not torch.isnan(dv).any()
    for i in range(b):
        sl = slice(i * s, (i + 1) * s)
        ref, ref_lse = _ref_attention(q[sl].float(), k[sl].float(), v[sl].float(), True, scale)
        assert (out[sl].float() - ref).abs().max().item() < 2e-2, ("out", i)
        assert (lse[:, sl] - ref_lse).abs().max().item() < 2e-2, ("lse", i)
        rq, rk, rv = _ref_grads(q[sl], k[sl], v[sl], do[sl], True, scale)
        assert _close(dv[sl], rv, 2e-2), ("dv", i)
        assert _close(dk[sl], rk, 2e-2), ("dk", i)
        assert _close(dq[sl], rq, 2e-2), ("dq", i)
    from astrai_b200.ops import native

    assert native.kernel_status(q.device) == 0


def test_flash_bwd_varlen_with_prefix():
    ops = _native()
    torch.manual_seed(3)
    d, hq, hkv = 128, 4, 2
    q_lens, k_lens = [130, 1, 77, 256], [130, 300, 200, 256]
    cu_q = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32, device="cuda")
    cu_k = torch.tensor([0] + list(torch.tensor(k_lens).cumsum(0)), dtype=torch.int32, device="cuda")
    q = torch.randn(sum(q_lens), hq, d, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(sum(k_lens), hkv, d, device="cuda", dtype=torch.bfloat16)
    v = torch.randn(sum(k_lens), hkv, d, device="cuda", dtype=torch.bfloat16)
    do = torch.randn_like(q)
    scale = 1.0 / math.sqrt(d)
    out, lse = ops.flash_fwd(q, k, v, cu_q, cu_k, 4, 0, 0, max(q_lens), True, scale)
    dq, dk, dv = ops.flash_bwd(q, k, v, out, do, lse, cu_q, cu_k, 4, 0, 0, max(q_lens), max(k_lens), True, scale)
    for i in range(4):
        qs = slice(int(cu_q[i]), int(cu_q[i + 1]))
        ks = slice(int(cu_k[i]), int(cu_k[i + 1]))
        rq, rk, rv = _ref_grads(q[qs], k[ks], v[ks], do[qs], True, scale)
        assert _close(dv[ks], rv, 2e-2), ("dv", i)
        assert _close(dk[ks], rk, 2e-2), ("dk", i)
        assert _close(dq[qs], rq, 2e-2), ("dq", i)


@pytest.mark.parametrize("page,hd,hq,hkv", [(16, 128, 8, 2), (8, 64, 4, 4), (64, 128, 4, 1), (32, 64, 6, 2)])
def test_paged_prefill_reads_the_pool_through_the_slot_table(page, hd, hq, hkv):
    """Ragged prefill over a paged pool (cached prefix + new tokens) without gathering the keys: against the fp32
    statement of causal attention per request, and bit-equal to the gather-then-varlen path."""
    from astrai_b200.ops import flash

    g = torch.Generator(device="cuda").manual_seed(page + hd)
    kv_lens, q_lens = [300, 77, 1025, page], [300, 13, 129, 1]      # full prefill, prefix + chunk, long prefix, one token
    n_pages_total = sum(-(-n // page) for n in kv_lens) + 7
    n_slots, max_ctx = n_pages_total * page, 1088
    k_pool = torch.randn(n_slots, hkv, hd, device="cuda", dtype=torch.bfloat16, generator=g)
    v_pool = torch.randn(n_slots, hkv, hd, device="cuda", dtype=torch.bfloat16, generator=g)
    perm = torch.randperm(n_pages_total, device="cuda", generator=g)
    table = torch.full((6, max_ctx), -1, dtype=torch.int32, device="cuda")
    rows = torch.tensor([4, 0, 2, 5], dtype=torch.int32, device="cuda")  # request rows are not in batch order
    used = 0
    for r, n in zip(rows.tolist(), kv_lens):
        pages = perm[used:used + -(-n // page)]
        used += pages.numel()
        slots = (pages[:, None] * page + torch.arange(page, device="cuda")[None]).reshape(-1).int()
        table[r, :slots.numel()] = slots  # whole pages are allocated, as the pool does
    cu_q = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32, device="cuda")
    cu_k = torch.tensor([0] + list(torch.tensor(kv_lens).cumsum(0)), dtype=torch.int32, device="cuda")
    q = torch.randn(sum(q_lens), hq, hd, device="cuda", dtype=torch.bfloat16, generator=g)
    out = flash.flash_attention_paged(q, k_pool, v_pool, cu_q, cu_k, table, rows, page, max(q_lens))
    gather = torch.cat([table[r, :n].long() for r, n in zip(rows.tolist(), kv_lens)])
    packed = flash.flash_attention_varlen(q, k_pool[gather], v_pool[gather], cu_q, cu_k, max(q_lens), max(kv_lens), causal=True)
    assert torch.equal(out, packed)
    at = 0
    for r, n, ql in zip(rows.tolist(), kv_lens, q_lens):
        slots = table[r, :n].long()
        kk = k_pool[slots].float().repeat_interleave(hq // hkv, dim=1)
        vv = v_pool[slots].float().repeat_interleave(hq // hkv, dim=1)
        qq = q[at:at + ql].float()
        s = torch.einsum("qhd,khd->hqk", qq, kk) * hd ** -0.5
        keep = torch.arange(n, device="cuda")[None, :] <= (n - ql + torch.arange(ql, device="cuda"))[:, None]
        s = s.masked_fill(~keep[None], float("-inf"))
        ref = torch.einsum("hqk,khd->qhd", torch.softmax(s, -1), vv)
        assert (out[at:at + ql].float() - ref).abs().max().item() < 2e-2
        at += ql
    from astrai_b200.ops import native

    assert native.kernel_status(torch.device("cuda")) == 0
