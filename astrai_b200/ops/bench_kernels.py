"""Kernel timing harness: ``python -m astrai_b200.ops.bench_kernels {gemm,skinny,flash,fp8,quant,sample,decode}``.

CUDA events on the launching stream, 3 warm-ups, median of N timed launches, a 256 MB buffer written between timed
launches to flush the 126 MB L2.  Library kernels (cuBLAS through ``torch.matmul``, cuDNN / flash through SDPA) are
timed next to ours as the reference point.  The numbers in ``profiles/`` come from these commands.
"""

from __future__ import annotations

import math
import sys

import torch


def _timer(flush_mb: int = 256):
    flush = torch.empty(flush_mb << 20, dtype=torch.uint8, device="cuda")

    def timeit(fn, n: int = 20) -> float:
        for _ in range(3):
            fn()
        ts = []
        for _ in range(n):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        ts.sort()
        return ts[len(ts) // 2]  # ms

    return timeit


def bench_gemm():
    from astrai_b200 import ops

    t = _timer()
    m = 8192
    print("bf16 GEMM, M = 8192 (TFLOP/s): ours fwd / dgrad / wgrad(fp32 accumulate) | cuBLAS fwd")
    for n, k, name in [(3072, 2048, "qkv"), (2048, 2048, "o_proj"), (11264, 2048, "gate+up"), (2048, 5632, "down"), (32000, 2048, "lm_head")]:
        x = torch.randn(m, k, device="cuda", dtype=torch.bfloat16)
        w = torch.randn(n, k, device="cuda", dtype=torch.bfloat16)
        dy = torch.randn(m, n, device="cuda", dtype=torch.bfloat16)
        acc = torch.zeros(n, k, device="cuda")
        fl = 2.0 * m * n * k / 1e9
        a = fl / t(lambda: ops.gemm(x, w))
        b = fl / t(lambda: ops.gemm(dy, w, b_kmajor=False))
        c = fl / t(lambda: ops.gemm(dy, x, out=acc, a_kmajor=False, b_kmajor=False, out_f32=True, accumulate=True))
        d = fl / t(lambda: torch.matmul(x, w.t()))
        print(f"  {n:6d} x {k:5d} ({name:8s}): {a:6.0f} / {b:6.0f} / {c:6.0f} | {d:6.0f}")


def bench_skinny():
    from astrai_b200 import ops

    t = _timer()
    print("decode-sized GEMM (GB/s of weight bytes): ours | cuBLAS")
    for m in (1, 16, 64, 128, 256):
        for n, k, name in [(3072, 2048, "qkv"), (2048, 2048, "o_proj"), (11264, 2048, "gate+up"), (2048, 5632, "down"), (32000, 2048, "lm_head")]:
            x = torch.randn(m, k, device="cuda", dtype=torch.bfloat16)
            w = torch.randn(n, k, device="cuda", dtype=torch.bfloat16)
            gb = n * k * 2 / 1e6
            a = gb / t(lambda: ops.gemm(x, w))
            b = gb / t(lambda: torch.matmul(x, w.t()))
            print(f"  M={m:3d} {n:6d} x {k:5d} ({name:8s}): {a:6.0f} | {b:6.0f}")


def bench_flash():
    import torch.nn.functional as F
    from torch.nn.attention import SDPBackend, sdpa_kernel

    from astrai_b200.ops import native

    native.require()
    op = torch.ops.astrai_b200
    t = _timer()
    b, s, hq, hkv, d = 4, 2048, 16, 4, 128
    q = torch.randn(b * s, hq, d, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(b * s, hkv, d, device="cuda", dtype=torch.bfloat16)
    v = torch.randn_like(k)
    do = torch.randn_like(q)
    sc = 1 / math.sqrt(d)
    fl = 4.0 * b * hq * s * s * d / 2 / 1e9  # causal forward GFLOP
    tf = t(lambda: op.flash_fwd(q, k, v, None, None, b, s, s, s, True, sc))
    out, lse = op.flash_fwd(q, k, v, None, None, b, s, s, s, True, sc)
    tb = t(lambda: op.flash_bwd(q, k, v, out, do, lse, None, None, b, s, s, s, s, True, sc))
    print(f"flash attention B{b} S{s} {hq}q/{hkv}kv D{d} causal")
    print(f"  ours : fwd {tf * 1e3:7.1f} us ({fl / tf:5.0f} TFLOP/s)  bwd {tb * 1e3:7.1f} us ({2.5 * fl / tb:5.0f} TFLOP/s at 5 GEMMs)")
    q4, k4, v4 = (x.view(b, s, -1, d).transpose(1, 2).detach().requires_grad_(True) for x in (q, k, v))
    with sdpa_kernel([SDPBackend.CUDNN_ATTENTION, SDPBackend.FLASH_ATTENTION], set_priority=True):
        tf2 = t(lambda: F.scaled_dot_product_attention(q4, k4, v4, is_causal=True, enable_gqa=True))
        o4 = F.scaled_dot_product_attention(q4, k4, v4, is_causal=True, enable_gqa=True)
        g4 = torch.randn_like(o4)
        tb2 = t(lambda: torch.autograd.grad(o4, (q4, k4, v4), g4, retain_graph=True))
    print(f"  SDPA : fwd {tf2 * 1e3:7.1f} us ({fl / tf2:5.0f} TFLOP/s)  bwd {tb2 * 1e3:7.1f} us ({2.5 * fl / tb2:5.0f} TFLOP/s)")
    print("  status", native.kernel_status(q.device))


def bench_fp8():
    from astrai_b200 import ops
    from astrai_b200.ops import fp8

    t = _timer()
    m = 8192
    print("fp8 GEMM, M = 8192 (TFLOP/s): ours fp8 | ours bf16 | quantise+transpose GB/s")
    for n, k in [(3072, 2048), (11264, 2048), (2048, 5632)]:
        x = torch.randn(m, k, device="cuda", dtype=torch.bfloat16)
        w = torch.randn(n, k, device="cuda", dtype=torch.bfloat16)
        one = torch.ones(1, device="cuda")
        xq, _, _ = fp8.quantize_bf16(x, one, "e4m3")
        wq, _, _ = fp8.quantize_bf16(w, one, "e4m3")
        fl = 2.0 * m * n * k / 1e9
        a = fl / t(lambda: fp8.mm_fp8(xq, wq, one, one))
        b = fl / t(lambda: ops.gemm(x, w))
        c = (m * k * 4) / 1e6 / t(lambda: fp8.quantize_bf16(x, one, "e4m3", with_transpose=True))
        print(f"  {n:6d} x {k:5d}: {a:6.0f} | {b:6.0f} | {c:6.0f}")


def bench_quant():
    """Block-scaled fp8 and int8 GEMMs next to the per-tensor fp8 and bf16 kernels."""
    from astrai_b200 import ops
    from astrai_b200.ops import fp8, fp8_block, int8

    t = _timer()
    m = 8192
    print("quantised GEMMs, M = 8192 (TFLOP/s or TOP/s): block fp8 | per-tensor fp8 | int8 | bf16 || act quantise GB/s: block fp8 | int8")
    for n, k in [(3072, 2048), (11264, 2048), (2048, 5632), (8192, 8192)]:
        x = torch.randn(m, k, device="cuda", dtype=torch.bfloat16)
        w = torch.randn(n, k, device="cuda", dtype=torch.bfloat16)
        one = torch.ones(1, device="cuda")
        xq, _, _ = fp8.quantize_bf16(x, one, "e4m3")
        wq, _, _ = fp8.quantize_bf16(w, one, "e4m3")
        xb, sa = fp8_block.quantize_act_block(x)
        wb, sb = fp8_block.quantize_weight_block(w)
        xi, si = int8.quantize_rows(x)
        wi, sw = int8.quantize_rows(w)
        fl = 2.0 * m * n * k / 1e9
        a = fl / t(lambda: fp8_block.mm_fp8_block(xb, sa, wb, sb))
        b = fl / t(lambda: fp8.mm_fp8(xq, wq, one, one))
        c = fl / t(lambda: int8.mm_int8(xi, si, wi, sw))
        d = fl / t(lambda: ops.gemm(x, w))
        e = (m * k * 3) / 1e6 / t(lambda: fp8_block.quantize_act_block(x))
        f = (m * k * 3) / 1e6 / t(lambda: int8.quantize_rows(x))
        print(f"  {n:6d} x {k:5d}: {a:6.0f} | {b:6.0f} | {c:6.0f} | {d:6.0f} || {e:6.0f} | {f:6.0f}")


def bench_sample():
    """The fused sampling kernel against the PyTorch pipeline (topk / sort / cumsum / scatter / multinomial)."""
    import importlib

    S = importlib.import_module("astrai_b200.inference.runtime.sample")
    t = _timer()
    print("sampling, top_k=50 top_p=0.9 temperature=0.8 (us per step): fused kernel | torch pipeline")
    for b, v in [(1, 100000), (16, 100000), (64, 100000), (256, 32000)]:
        logits = torch.randn(b, v, device="cuda", dtype=torch.bfloat16) * 2
        temps = torch.full((b,), 0.8, device="cuda")
        ks = torch.full((b,), 50, device="cuda", dtype=torch.int32)
        ps = torch.full((b,), 0.9, device="cuda")
        hints = {"max_k": 50, "top_p_active": True, "has_freq": False, "greedy": False}
        gen = torch.Generator(device="cuda").manual_seed(1)
        fused = t(lambda: S.sample(logits, temps, ks, ps, hints=hints))
        plain = t(lambda: S.sample(logits, temps, ks, ps, hints=hints, generator=gen))
        print(f"  B={b:3d} V={v:6d}: {fused * 1e3:7.1f} | {plain * 1e3:7.1f}")


def bench_decode():
    t = _timer()
    op = torch.ops.astrai_b200
    from astrai_b200.ops import native

    native.require()
    print("paged decode attention (GB/s of K/V bytes), page 16; heads q/kv, head dim")
    for b, ctx, hq, hkv, d in [(1, 4096, 16, 4, 128), (16, 2048, 16, 4, 128), (64, 2048, 16, 4, 128), (64, 8192, 16, 4, 128),
                               (16, 1152, 24, 4, 64), (64, 2048, 24, 4, 64)]:
        n_slots = b * ctx + 1024
        kb = torch.randn(n_slots, hkv, d, device="cuda", dtype=torch.bfloat16)
        vb = torch.randn_like(kb)
        table = torch.arange(b * ctx, dtype=torch.int32, device="cuda").view(b, ctx)
        rows = torch.arange(b, dtype=torch.int32, device="cuda")
        seq = torch.full((b,), ctx, dtype=torch.long, device="cuda")
        q = torch.randn(b, hq, d, device="cuda", dtype=torch.bfloat16)
        o_part = torch.zeros(b, hq, 32, d, device="cuda")
        ml = torch.zeros(b, hq, 32, 2, device="cuda")
        cnt = torch.zeros(b * hkv, dtype=torch.int32, device="cuda")
        out = torch.empty_like(q)
        splits = int(op.paged_decode_splits(b, hkv, ctx, 32))
        ms = t(lambda: op.paged_decode_(q, kb, vb, table, rows, seq, d ** -0.5, splits, o_part, ml, cnt, out))
        gb = 2 * b * ctx * hkv * d * 2 / 1e6
        if "--sweep" in sys.argv:
            sweep = {sp: t(lambda: op.paged_decode_(q, kb, vb, table, rows, seq, d ** -0.5, sp, o_part, ml, cnt, out), n=8)
                     for sp in (1, 2, 3, 4, 6, 8, 10, 12, 16, 24, 32) if sp * 128 <= ctx * 2}
            print("    splits sweep (us): " + "  ".join(f"{sp}:{v * 1e3:.1f}" for sp, v in sweep.items()))
        print(f"  B={b:3d} ctx={ctx:5d} {hq}q/{hkv}kv D{d} splits={splits:2d}: {ms * 1e3:7.1f} us  {gb / ms:6.0f} GB/s")


if __name__ == "__main__":
    table = {"gemm": bench_gemm, "skinny": bench_skinny, "flash": bench_flash, "fp8": bench_fp8, "quant": bench_quant, "sample": bench_sample, "decode": bench_decode}
    which = [a for a in sys.argv[1:] if not a.startswith("--")] or list(table)
    for name in which:
        table[name]()
