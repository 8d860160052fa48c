"""One launch of every kernel of the library on a profiling-sized case: ``python -m astrai_b200.ops.profile_kernels``.

Meant to run under ``ncu`` (one or a few launches of each kernel, device footprint well under a few GB, inputs of the
memory-bound kernels larger than the 126 MB L2 so that DRAM figures mean something).  Several ranks of the
communication kernels are emulated on one GPU with preset flags (no kernel waits for another).
"""

from __future__ import annotations

import math

import torch


def main():
    from astrai_b200 import ops
    from astrai_b200.ops import fp8, native
    from astrai_b200.parallel.symm import LocalArena

    native.require()
    op = torch.ops.astrai_b200
    dev = torch.device("cuda")
    torch.manual_seed(0)
    bf = dict(device=dev, dtype=torch.bfloat16)

    # ---- GEMMs (one micro-batch of the 1B model: 8192 tokens)
    m, d, f = 8192, 2048, 5632
    x = torch.randn(m, d, **bf)
    w_gu = torch.randn(2 * f, d, **bf) * 0.02
    y = ops.gemm(x, w_gu)                                           # 2-CTA forward
    dy = torch.randn(m, 2 * f, **bf)
    ops.gemm(dy, w_gu, b_kmajor=False)                              # dgrad (MN-major B)
    acc = torch.zeros(2 * f, d, device=dev)
    ops.gemm(dy, x, out=acc, a_kmajor=False, b_kmajor=False, out_f32=True, accumulate=True)  # wgrad, fp32 accumulate
    ops.gemm(x[:128], w_gu)                                         # 1-CTA kernel (M < 256)
    ops.gemm(x[:16], w_gu)                                          # skinny, cluster split-K
    one = torch.ones(1, device=dev)
    xq, xqt, _ = fp8.quantize_bf16(x, one, "e4m3", with_transpose=True)
    wq, _, _ = fp8.quantize_bf16(w_gu, one, "e4m3")
    fp8.mm_fp8(xq, wq, one, one)

    # ---- elementwise / normalisation / loss / optimizer on > L2 inputs (64 k tokens x 2048 = 268 MB bf16)
    big = torch.randn(65536, d, **bf, requires_grad=True)
    wn = torch.ones(d, **bf, requires_grad=True)
    out = ops.rms_norm(big, wn, 1e-6)
    out.backward(torch.randn_like(out))
    gu = torch.randn(32768, 2 * f, **bf, requires_grad=True)
    s = ops.swiglu_fused(gu)
    s.backward(torch.randn_like(s))
    qkv = torch.randn(65536, (16 + 8) * 128, **bf, requires_grad=True)
    pos = torch.arange(65536, device=dev) % 2048
    inv = 1.0 / (10000 ** (torch.arange(0, 128, 2, device=dev).float() / 128))
    ang = pos[:, None].float() * inv[None]
    freqs = torch.stack([ang.cos(), ang.sin()], dim=-1)
    q, k, v = ops.qkv_rope(qkv, freqs, 16, 4, 128)
    (q.sum() + k.sum()).backward()
    table = torch.randn(32000, d, **bf, requires_grad=True)
    ids = torch.randint(0, 32000, (65536,), device=dev)
    e = ops.embedding(ids, table)
    e.backward(torch.randn_like(e))
    h = torch.randn(8192, d, **bf, requires_grad=True)
    lm = (torch.randn(32000, d, **bf) * 0.02).requires_grad_(True)
    loss = ops.linear_cross_entropy(h, lm, ids[:8192], 0.05)
    loss.backward()
    n = 128 << 20
    p, g = torch.randn(n, **bf), torch.randn(n, device=dev)
    m1, m2, master = torch.zeros(n, device=dev), torch.zeros(n, device=dev), p.float()
    ss = ops.sumsq(g)
    coef, _ = ops.clip_coef(ss, 1.0)
    ops.adamw_(p, g, m1, m2, lr=1e-4, betas=(0.9, 0.999), weight_decay=0.1, step=1, master=master, grad_scale=coef)
    del p, g, m1, m2, master, big, gu, qkv

    # ---- attention
    b, sl, hq, hkv, hd = 4, 2048, 16, 4, 128
    qa = torch.randn(b * sl, hq, hd, **bf)
    ka = torch.randn(b * sl, hkv, hd, **bf)
    va = torch.randn_like(ka)
    o, lse = op.flash_fwd(qa, ka, va, None, None, b, sl, sl, sl, True, 1 / math.sqrt(hd))
    op.flash_bwd(qa, ka, va, o, torch.randn_like(o), lse, None, None, b, sl, sl, sl, sl, True, 1 / math.sqrt(hd))
    nb, ctx = 64, 4096
    kb = torch.randn(nb * ctx, hkv, hd, **bf)
    vb = torch.randn_like(kb)
    tbl = torch.arange(nb * ctx, dtype=torch.int32, device=dev).view(nb, ctx)
    rows = torch.arange(nb, dtype=torch.int32, device=dev)
    seq = torch.full((nb,), ctx, dtype=torch.long, device=dev)
    qd = torch.randn(nb, hq, hd, **bf)
    o_part, ml = torch.zeros(nb, hq, 32, hd, device=dev), torch.zeros(nb, hq, 32, 2, device=dev)
    cnt = torch.zeros(nb * hkv, dtype=torch.int32, device=dev)
    od = torch.empty_like(qd)
    op.paged_decode_(qd, kb, vb, tbl, rows, seq, hd ** -0.5, int(op.paged_decode_splits(nb, hkv, ctx, 32)), o_part, ml, cnt, od)
    op.kv_append_(torch.randn(nb, hkv, hd, **bf), torch.randn(nb, hkv, hd, **bf), kb, vb, torch.arange(nb, dtype=torch.int32, device=dev))

    # ---- communication kernels, two emulated ranks on this GPU (flags preset: nothing waits)
    world, n_shard = 2, 32 << 20
    arena = LocalArena(world * n_shard * 6 + (1 << 20), world, dev)
    bufs = []
    for r in range(world):
        a = arena.view(r)
        bufs.append((a.alloc(world * n_shard, torch.float32), a.alloc(world * n_shard, torch.bfloat16), a.alloc_flags(16)))
        bufs[r][2].tensor.fill_(1)
    grad, param, flags = bufs[0]
    red, sq = torch.empty(n_shard, device=dev), torch.zeros(1, device=dev)
    op.fsdp_reduce_scatter_(grad.peer_ptrs, 0, flags.peer_ptrs, 0, 0, red, sq, 0, 16, 1, 0.5, 64)
    mm, vv, ms = torch.zeros(n_shard, device=dev), torch.zeros(n_shard, device=dev), torch.zeros(n_shard, device=dev)
    op.fsdp_adamw_allgather_(param.peer_ptrs, 0, flags.peer_ptrs, 0, 0, ms, red, mm, vv, 1e-4, 0.9, 0.999, 1e-8, 0.1, 1, None, 0, 16, 2,
                             torch.zeros(1, dtype=torch.int32, device=dev), 128)
    del arena, bufs
    mt, kt, nt = 2048, 2048, 4096
    arena = LocalArena(mt * kt * 2 + world * (mt // world) * nt * 2 + (2 << 20), world, dev)
    xs, st, fl = [], [], []
    for r in range(world):
        a = arena.view(r)
        xs.append(a.alloc(mt * kt, torch.bfloat16))
        st.append(a.alloc(world * (mt // world) * nt, torch.bfloat16))
        fl.append(a.alloc_flags(64))
        xs[r].tensor.normal_()
        fl[r].tensor.fill_(1)
    wt = torch.randn(nt, kt, **bf) * 0.02
    yt = torch.empty(mt, nt, **bf)
    z8 = lambda: torch.zeros(8, dtype=torch.int32, device=dev)
    op.tp_gemm_allgather_(xs[0].peer_ptrs, wt, True, yt, fl[0].peer_ptrs, z8(), z8(), 0, 0, 64, 1, 0.5, 16)
    outr = torch.empty(mt // world, nt, **bf)
    op.tp_gemm_reducescatter_(xs[0].tensor.view(mt, kt), wt, True, st[0].peer_ptrs, outr, fl[0].peer_ptrs, z8(), 0, 1, 64, 1, 0.5, False)
    op.tp_reduce_(st[0].tensor, outr, world)
    del arena, xs, st, fl

    # ---- quantised GEMMs, sampling, decode with 6 query heads per kv head
    from astrai_b200.ops import fp8_block, int8, moe

    xb, sa = fp8_block.quantize_act_block(x)
    wb, sb = fp8_block.quantize_weight_block(w_gu)
    fp8_block.mm_fp8_block(xb, sa, wb, sb)
    xi, si = int8.quantize_rows(x)
    wi, sw = int8.quantize_rows(w_gu)
    int8.mm_int8(xi, si, wi, sw)
    logits = torch.randn(64, 100000, **bf)
    op.sample_rows(logits, torch.full((64,), 0.8, device=dev), torch.full((64,), 50, device=dev, dtype=torch.int32),
                   torch.full((64,), 0.9, device=dev), None, None, None, False, 1, 1)
    hq6, hkv6, hd6, nb6, ctx6 = 24, 4, 64, 16, 1152
    kb6 = torch.randn(nb6 * ctx6, hkv6, hd6, **bf)
    vb6 = torch.randn_like(kb6)
    tbl6 = torch.arange(nb6 * ctx6, dtype=torch.int32, device=dev).view(nb6, ctx6)
    qd6 = torch.randn(nb6, hq6, hd6, **bf)
    op.paged_decode_(qd6, kb6, vb6, tbl6, torch.arange(nb6, dtype=torch.int32, device=dev),
                     torch.full((nb6,), ctx6, dtype=torch.long, device=dev), hd6 ** -0.5,
                     int(op.paged_decode_splits(nb6, hkv6, ctx6, 32)), torch.zeros(nb6, hq6, 32, hd6, device=dev),
                     torch.zeros(nb6, hq6, 32, 2, device=dev), torch.zeros(nb6 * hkv6, dtype=torch.int32, device=dev),
                     torch.empty_like(qd6))

    # ---- mixture of experts: router, plan, permute, grouped GEMMs (forward, dgrad, ragged-K wgrad), combine
    t_moe, e_moe, k_moe, f_moe = 8192, 16, 4, 1408
    xm = torch.randn(t_moe, d, **bf, requires_grad=True)
    router = torch.randn(e_moe, d, **bf) * 0.1
    w1 = (torch.randn(e_moe, 2 * f_moe, d, **bf) * 0.02).requires_grad_(True)
    w2 = (torch.randn(e_moe, d, f_moe, **bf) * 0.02).requires_grad_(True)
    _p, idx, wts, counts, _s = moe.route(ops.gemm(xm.detach(), router), k_moe, True)
    xs_m, plan = moe.dispatch(xm, idx, counts, e_moe)
    hm = ops.swiglu_fused(moe.zero_unused_rows(moe.grouped_linear(xs_m, w1, plan), plan))
    ym = moe.zero_unused_rows(moe.grouped_linear(hm, w2, plan), plan)
    moe.combine(ym, wts, plan).backward(torch.randn(t_moe, d, **bf))

    # ---- context-parallel attention, rank 0 of two emulated ranks (K / V gathered by the copy CTAs of the launch)
    from astrai_b200.parallel import context_parallel as cpar

    wcp, ccp, bcp, hqc, hkc, dcp = 2, 2048, 1, 16, 4, 128
    scp, rowc = 2 * wcp * ccp, hkc * dcp
    arena = LocalArena(cpar.arena_bytes_for(bcp, scp, wcp, hkc, dcp), wcp, dev)
    cxs = [cpar.CPContext(arena.view(r), r, wcp, timeout_s=0.5) for r in range(wcp)]
    srcs = [cx.kv_source(bcp, ccp, rowc, 1) for cx in cxs]
    stages = [cx.stage(bcp, ccp, rowc, 0) for cx in cxs]
    for r, cx in enumerate(cxs):
        srcs[r].tensor.normal_()
        cx.flags.tensor.fill_(1)
    qc = torch.randn(bcp * 2 * ccp, hqc, dcp, **bf)
    kf, vf = torch.zeros(bcp * scp, hkc, dcp, **bf), torch.zeros(bcp * scp, hkc, dcp, **bf)
    oc, lsec = op.cp_flash_fwd(qc, kf, vf, bcp, ccp, wcp, 0, dcp ** -0.5, srcs[0].peer_ptrs, cxs[0].flags.peer_ptrs, 0, 1, 1, 8,
                               cxs[0].chunk_state, 0.5)
    op.cp_flash_bwd(qc, kf, vf, oc, torch.randn_like(oc), lsec, bcp, ccp, wcp, 0, dcp ** -0.5, stages[0].peer_ptrs,
                    cxs[0].flags.peer_ptrs, 0, 1, 2, cxs[0].tile_counter, 0.5)
    torch.cuda.synchronize()
    print("status", native.kernel_status(dev), "launches", native.launch_count())


if __name__ == "__main__":
    main()
