"""Achieved fraction of the roofline for every fused compute + collective path, next to its library-collective arm.

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 -m astrai_b200.parallel.bench_fused \\
        [--ops tp_ag,tp_rs,cp,ep,fsdp] [--iters 10] [--out fused.json]

For each path the fused kernel (``p2p``) and the same math around NCCL collectives (``nccl``) run on the shapes of the
configurations they serve; each timing is CUDA events on the launching stream after warm-up, maximum over the ranks.
The roofline of a path is the slower of its FLOPs at the measured sustained bf16 rate and the bytes one rank must
receive over NVLink at the measured peer-copy rate:

    t_roof = max(FLOPs / 1378.7 TFLOP/s, bytes / 770 GB/s)        fraction = t_roof / t_measured

* ``tp_ag`` / ``tp_rs``: all-gather -> GEMM and GEMM -> reduce-scatter of the 8B model's MLP (gate|up, down) and
  attention (q|k|v, o_proj) projections under tensor parallelism with sequence-sharded activations (65 536 tokens per
  step); the attention projections have a quarter of the MLP's FLOPs for the same bytes, so they are NVLink-bound;
* ``cp``: causal attention forward + backward of one 65 536-token sequence sharded zig-zag over the ranks (32 query / 8 kv
  heads of 128);
* ``ep``: one MoE layer forward + backward (8 192 tokens per rank, 64 experts, top-6, hidden 2048, expert FFN 1408);
* ``fsdp``: reduce-scatter (+ squared norm), clip, AdamW and parameter all-gather of one 1B-model decoder block
  (45.1 M parameters) as the optimizer step runs them.

The reference has no such path to compare with (it only calls ``torch.distributed`` collectives,
``astrai/parallel/executor.py:254-428``); the ``nccl`` arm is the baseline.
"""

from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

PEAK_FLOPS = 1378.7e12   # measured sustained bf16 GEMM rate of this pool's B200
LINK_BPS = 770e9         # measured peer copy, per direction per GPU


def _time(fn, iters, warm=3):
    for _ in range(warm):
        fn()
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def _row(name, what, flops, link_bytes, ms):
    roof = max(flops / PEAK_FLOPS, link_bytes / LINK_BPS) * 1e3
    out = {"path": name, "shape": what, "tflop": round(flops / 1e12, 3), "nvlink_mb_per_rank": round(link_bytes / 1e6, 1),
           "roofline_ms": round(roof, 3), "bound": "compute" if flops / PEAK_FLOPS >= link_bytes / LINK_BPS else "nvlink"}
    for arm, v in ms.items():
        out[f"{arm}_ms"] = round(v, 3)
        out[f"{arm}_fraction_of_roofline"] = round(roof / v, 3)
    return out


def bench_tp(world, rank, dev, iters, which, slots=(0,)):
    from astrai_b200.parallel import tensor_parallel as tpar

    m, d, ffn = 65536, 4096, 14336
    ms_rows = m // world
    ctx = tpar.init_tensor_parallel(4 << 30, timeout_s=60.0)
    g = torch.Generator(device="cuda").manual_seed(rank)
    rows = []
    qkv = (32 + 8 + 8) * 128  # 32 query and 8 + 8 key / value heads of 128
    if which == "tp_ag":
        x = torch.randn(ms_rows, d, device=dev, dtype=torch.bfloat16, generator=g)
        for name, n in (("gate|up forward", 2 * ffn // world), ("q|k|v forward", qkv // world)):
            w = torch.randn(n, d, device=dev, dtype=torch.bfloat16, generator=g) * 0.02
            ms = {"nccl": _time(lambda: tpar.allgather_gemm(x, w, True, ctx=ctx, comm="nccl"), iters)}
            for sl in slots:  # 0: the launcher's own choice; 1..3: forced number of copy slots
                ctx.copy_slots = sl
                ms["p2p" if sl == 0 else f"p2p_slots{sl}"] = _time(lambda: tpar.allgather_gemm(x, w, True, ctx=ctx, comm="p2p"), iters)
            ctx.copy_slots = 0
            rows.append(_row(f"TP all-gather -> GEMM ({name})", f"[{m}x{d}] x [{n}x{d}]^T, tp{world}",
                             2.0 * m * n * d, (world - 1) / world * m * d * 2, ms))
    else:
        for name, k in (("down forward", ffn // world), ("o_proj forward", d // world)):
            x = torch.randn(m, k, device=dev, dtype=torch.bfloat16, generator=g)
            w = torch.randn(d, k, device=dev, dtype=torch.bfloat16, generator=g) * 0.02
            ms = {"nccl": _time(lambda: tpar.gemm_reducescatter(x, w, True, ctx=ctx, comm="nccl"), iters)}
            for sl in slots:
                ctx.copy_slots = sl
                ms["p2p" if sl == 0 else f"p2p_slots{sl}"] = _time(lambda: tpar.gemm_reducescatter(x, w, True, ctx=ctx, comm="p2p"), iters)
            ctx.copy_slots = 0
            rows.append(_row(f"TP GEMM -> reduce-scatter ({name})", f"[{m}x{k}] x [{d}x{k}]^T, tp{world}",
                             2.0 * m * d * k, (world - 1) / world * m * d * 2, ms))
    tpar.set_context(None)
    return rows


def bench_cp(world, rank, dev, iters):
    from astrai_b200.parallel import context_parallel as cpar

    b, s, hq, hkv, hd = 1, 65536, 32, 8, 128
    cp = cpar.init_context_parallel(cpar.arena_bytes_for(b, s, world, hkv, hd), timeout_s=60.0)
    g = torch.Generator(device="cuda").manual_seed(rank)
    local = s // world
    q = torch.randn(b, local, hq, hd, device=dev, dtype=torch.bfloat16, generator=g)
    k = torch.randn(b, local, hkv, hd, device=dev, dtype=torch.bfloat16, generator=g)
    v = torch.randn(b, local, hkv, hd, device=dev, dtype=torch.bfloat16, generator=g)
    do = torch.randn_like(q)

    def step(comm):
        ql, kl, vl = (t.detach().requires_grad_(True) for t in (q, k, v))
        cpar.ring_attention(ql, kl, vl, ctx=cp, comm=comm).backward(do)

    ms = {c: _time(lambda c=c: step(c), iters) for c in ("nccl", "p2p")}
    flops = 3.5 * (4.0 * s * s * hq * hd / 2) / world          # causal forward + backward (2.5x), this rank's share
    kv_bytes = (world - 1) / world * s * hkv * hd * 2 * 2        # K and V of the other ranks, bf16
    link = 2 * kv_bytes                                          # gathered in forward, dK / dV returned in backward
    cpar.set_context(None)
    return [_row("CP attention forward + backward (K/V gather and dK/dV return inside the kernels)",
                 f"S {s}, {hq}q/{hkv}kv x {hd}, cp{world}", flops, link, ms)]


def bench_ep(world, rank, dev, iters):
    from astrai_b200.ops import functional as F
    from astrai_b200.ops import moe
    from astrai_b200.parallel import expert_parallel as epar

    t, h, f, e, k = 8192, 2048, 1408, 64, 6
    epar.init_expert_parallel(epar.arena_bytes_for(t, h, k, world, e, 2.0), timeout_s=60.0)
    g = torch.Generator(device="cuda").manual_seed(100 + rank)
    local = e // world
    router = (torch.randn(e, h, device=dev, generator=g) * 0.02).bfloat16()
    gate_up = (torch.randn(local, 2 * f, h, device=dev, generator=g) * 0.02).bfloat16().requires_grad_(True)
    down = (torch.randn(local, h, f, device=dev, generator=g) * 0.02).bfloat16().requires_grad_(True)
    x0 = torch.randn(t, h, device=dev, generator=g).bfloat16()
    dout = torch.randn(t, h, device=dev, generator=g).bfloat16()

    def step(comm):
        x = x0.detach().requires_grad_(True)
        _p, idx, wts, counts, _s = moe.route(F.linear(x, router), k, True)
        if comm == "p2p":
            out = epar.ep_experts(x, idx, wts, counts, gate_up, down, capacity_factor=2.0)
        else:
            out = epar.ep_experts_collective(x, idx, wts, counts, gate_up, down)
        out.backward(dout)
        gate_up.grad = down.grad = None

    ms = {c: _time(lambda c=c: step(c), iters) for c in ("nccl", "p2p")}
    flops = 3.0 * t * k * 3 * 2.0 * h * f                        # three expert matrices, forward + backward (3x)
    link = 4 * (world - 1) / world * t * k * h * 2               # dispatch and combine, forward and backward, bf16 rows
    epar.set_context(None)
    return [_row("EP MoE layer forward + backward (dispatch / combine inside the grouped GEMMs)",
                 f"{t} tokens/rank, {e} experts top-{k}, hidden {h}, ffn {f}, ep{world}", flops, link, ms)]


def bench_fsdp(world, rank, dev, iters):
    """One decoder block of the 1B model through the fused reduce-scatter and the fused AdamW + all-gather kernels."""
    from astrai_b200.optim import FusedAdamW
    from astrai_b200.parallel import ExecutorFactory

    rows = []
    numel = 45_092_864
    res = {}
    for comm in ("nccl", "p2p"):
        model = torch.nn.Linear(numel // 2048, 2048, bias=False).to(dev, torch.bfloat16)  # one flat unit of that size
        holder = torch.nn.ModuleList([model])
        wrapper = torch.nn.Module()
        wrapper.layers = holder
        ex = ExecutorFactory.create("fsdp", grad_accum_steps=1, comm=comm, comm_timeout_s=20.0)
        wrapped, opt, _ = ex.prepare(lambda: wrapper, lambda m: FusedAdamW(m.parameters(), lr=1e-4))
        unit = ex.engine.units[0]
        unit.grad_buf.normal_()

        def update():
            ex._reduce_unit(unit)
            ex._finish_reductions()
            ex.clip_grad_norm(wrapped, 1.0)
            opt.step()
            ex._wait_all_gathers()

        res[comm] = _time(update, iters)
        del ex, opt, wrapped
        torch.cuda.synchronize()
    shard = numel / world
    rows.append(_row("FSDP step of one 1B decoder block: gradient reduce-scatter (+ norm), clip, AdamW, parameter all-gather",
                     f"{numel} parameters (fp32 gradients in, bf16 parameters out), fsdp{world}", 0.0,
                     (world - 1) * shard * 4 + (world - 1) * shard * 2, res))
    return rows


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--ops", default="tp_ag,tp_rs,cp,ep,fsdp")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--out", default=None)
    ap.add_argument("--tp-slots", default="0", help="tp_ag / tp_rs: comma list of copy-slot counts to time (0 = the launcher's choice)")
    args = ap.parse_args(argv)
    from astrai_b200.ops import native
    from astrai_b200.parallel.setup import setup_parallel

    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ.get("LOCAL_RANK", 0))
    rows = []
    with setup_parallel(rank, world, local, "nccl", os.environ.get("MASTER_ADDR", "127.0.0.1"),
                        os.environ.get("MASTER_PORT", "29540"), "cuda"):
        dev = torch.device("cuda", local)
        native.require()
        for op in args.ops.split(","):
            try:
                if op in ("tp_ag", "tp_rs"):
                    rows += bench_tp(world, rank, dev, args.iters, op, tuple(int(v) for v in args.tp_slots.split(",")))
                elif op == "cp":
                    rows += bench_cp(world, rank, dev, args.iters)
                elif op == "ep":
                    rows += bench_ep(world, rank, dev, args.iters)
                elif op == "fsdp":
                    rows += bench_fsdp(world, rank, dev, args.iters)
            except Exception as exc:  # noqa: BLE001 - one path failing must not lose the others' numbers
                rows.append({"path": op, "error": f"{type(exc).__name__}: {exc}"[:300]})
            torch.cuda.synchronize()
            torch.cuda.empty_cache()
        status = native.kernel_status(dev)
    if rank == 0:
        doc = {"n_gpus": world, "peak_tflops": PEAK_FLOPS / 1e12, "link_gb_s": LINK_BPS / 1e9, "kernel_status": status, "rows": rows}
        text = json.dumps(doc, indent=1)
        print(text)
        if args.out:
            with open(args.out, "w") as fh:
                fh.write(text + "\n")
    return 0


if __name__ == "__main__":
    sys.exit(main())
