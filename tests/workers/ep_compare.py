"""Worker of the multi-GPU expert-parallel test: an ``EPMoE`` layer (experts sharded over the ranks, rows moved by the
fused gather / scatter GEMMs) against the single-GPU grouped-GEMM path run with ALL experts on every rank's own tokens;
forward output, input gradient, and (after summing the single-GPU weight gradients over ranks) the gradients of this
rank's experts and of the router.  With ``--time`` also the device time per forward + backward (max over ranks).
Launched by torchrun."""

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", required=True)
    ap.add_argument("--tokens", type=int, default=512)
    ap.add_argument("--hidden", type=int, default=256)
    ap.add_argument("--inter", type=int, default=128)
    ap.add_argument("--experts", type=int, default=8)
    ap.add_argument("--top-k", type=int, default=2)
    ap.add_argument("--time", type=int, default=0)
    args = ap.parse_args()
    from astrai_b200.ops import functional as F
    from astrai_b200.ops import moe, native
    from astrai_b200.parallel import expert_parallel as epar
    from astrai_b200.parallel.setup import setup_parallel

    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    with setup_parallel(rank, world, local, "nccl", os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"], "cuda"):
        dev = torch.device("cuda", local)
        native.require()
        t, h, f, e, k = args.tokens, args.hidden, args.inter, args.experts, args.top_k
        ep = epar.init_expert_parallel(epar.arena_bytes_for(t, h, k, world, e), timeout_s=30.0)
        g = torch.Generator(device="cpu").manual_seed(5)
        router = (torch.randn(e, h, generator=g) * 0.1).bfloat16().to(dev)
        gate_up = (torch.randn(e, 2 * f, h, generator=g) * 0.05).bfloat16().to(dev)
        down = (torch.randn(e, h, f, generator=g) * 0.05).bfloat16().to(dev)
        xs = [torch.randn(t, h, generator=g).bfloat16() for _ in range(world)]
        douts = [torch.randn(t, h, generator=g).bfloat16() for _ in range(world)]
        x_mine, dout = xs[rank].to(dev), douts[rank].to(dev)

        layer = epar.EPMoE(h, f, e, k, world, rank, dtype=torch.bfloat16, device=dev)
        with torch.no_grad():
            layer.router.copy_(router)
            layer.gate_up.copy_(epar.EPMoE.shard(gate_up, world, rank))
            layer.down.copy_(epar.EPMoE.shard(down, world, rank))
        got = None
        for _ in range(3):  # several calls: buffer parity and epochs advance
            layer.zero_grad()
            x = x_mine.clone().requires_grad_(True)
            out = layer(x)
            out.backward(dout)
            got = (out.detach().float(), x.grad.float(), layer.gate_up.grad.float().clone(), layer.down.grad.float().clone(),
                   layer.router.grad.float().clone())

        # single-GPU path with every expert, on this rank's tokens
        r2, gu2, dn2 = (p.clone().requires_grad_(True) for p in (router, gate_up, down))
        x2 = x_mine.clone().requires_grad_(True)
        logits = F.linear(x2, r2)
        _probs, idx, wts, counts, _psum = moe.route(logits, k, True)
        xs_sorted, plan = moe.dispatch(x2, idx, counts, e)
        hh = F.swiglu_fused(moe.zero_unused_rows(moe.grouped_linear(xs_sorted, gu2, plan), plan))
        yy = moe.zero_unused_rows(moe.grouped_linear(hh, dn2, plan), plan)
        ref_out = moe.combine(yy, wts, plan)
        ref_out.backward(dout)
        wg = [gu2.grad.float(), dn2.grad.float()]
        for w_ in wg:
            dist.all_reduce(w_)
        el = e // world
        refs = (ref_out.detach().float(), x2.grad.float(), wg[0][rank * el:(rank + 1) * el], wg[1][rank * el:(rank + 1) * el],
                r2.grad.float())
        names = ("out", "dx", "d_gate_up", "d_down", "d_router")
        diffs = {n: float((a - b).abs().max() / (b.abs().max() + 1e-6)) for n, a, b in zip(names, got, refs)}
        if args.time:
            x = x_mine.clone().requires_grad_(True)
            dist.barrier()
            torch.cuda.synchronize()
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
            ev[0].record()
            for _ in range(args.time):
                out = layer(x)
                out.backward(dout)
                x.grad = None
            ev[1].record()
            torch.cuda.synchronize()
            tm = torch.tensor([ev[0].elapsed_time(ev[1]) / args.time], device=dev)
            dist.all_reduce(tm, op=dist.ReduceOp.MAX)
            diffs["ms"] = float(tm.item())
            # the same rows through the single-GPU path (all experts local, no transfer): what the exchange costs
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
            torch.cuda.synchronize()
            ev[0].record()
            for _ in range(args.time):
                logits = F.linear(x, r2)
                _p, idx, wts, counts, _s = moe.route(logits, k, True)
                xs_sorted, plan = moe.dispatch(x, idx, counts, e)
                hh = F.swiglu_fused(moe.zero_unused_rows(moe.grouped_linear(xs_sorted, gu2, plan), plan))
                yy = moe.zero_unused_rows(moe.grouped_linear(hh, dn2, plan), plan)
                moe.combine(yy, wts, plan).backward(dout)
                x.grad = None
            ev[1].record()
            torch.cuda.synchronize()
            tm = torch.tensor([ev[0].elapsed_time(ev[1]) / args.time], device=dev)
            dist.all_reduce(tm, op=dist.ReduceOp.MAX)
            diffs["ms_all_experts_local"] = float(tm.item())
        diffs["status"] = native.kernel_status(dev)
        gathered = [None] * world
        dist.all_gather_object(gathered, diffs)
        if rank == 0:
            with open(args.out, "w") as fh:
                json.dump(gathered, fh)


if __name__ == "__main__":
    main()
