"""Worker of the multi-GPU context-parallel attention test: the zig-zag-sharded causal attention run forward +
backward with the fused peer-memory kernels (``p2p``) and with NCCL all-gather / reduce-scatter around the same
kernels, both compared with fp32 PyTorch attention of the whole sequence; with ``--time`` it also reports the device
time of forward + backward per call (max over ranks).  Launched by torchrun."""

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
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--batch", type=int, default=2)
    ap.add_argument("--heads", type=int, default=8)
    ap.add_argument("--kv-heads", type=int, default=4)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--time", type=int, default=0, help="timed iterations per mode (0: correctness only)")
    ap.add_argument("--no-check", action="store_true", help="skip the fp32 reference (long sequences)")
    args = ap.parse_args()
    from astrai_b200.ops import native
    from astrai_b200.parallel import context_parallel as cpar
    from astrai_b200.parallel.setup import setup_parallel

    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    with setup_parallel(rank, world, local, "nccl", os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"], "cuda"):
        dev = torch.device("cuda", local)
        native.require()
        b, s, hq, hkv, d = args.batch, args.seq, args.heads, args.kv_heads, args.head_dim
        cp = cpar.init_context_parallel(cpar.arena_bytes_for(b, s, world, hkv, d), timeout_s=30.0)
        g = torch.Generator(device="cpu").manual_seed(7)  # same tensors on every rank
        q = torch.randn(b, s, hq, d, generator=g).bfloat16()
        k = torch.randn(b, s, hkv, d, generator=g).bfloat16()
        v = torch.randn(b, s, hkv, d, generator=g).bfloat16()
        do = torch.randn(b, s, hq, d, generator=g).bfloat16()
        mine = [cpar.zigzag_split(t, world, rank).to(dev) for t in (q, k, v, do)]
        res, times = {}, {}
        for comm in ("nccl", "p2p"):
            outs = None
            for _ in range(3):  # several calls: buffer parity and epochs advance
                ql, kl, vl = (t.clone().requires_grad_(True) for t in mine[:3])
                out = cpar.ring_attention(ql, kl, vl, ctx=cp, comm=comm)
                out.backward(mine[3])
                outs = (out.detach().float(), ql.grad.float(), kl.grad.float(), vl.grad.float())
            res[comm] = outs
            if args.time:
                ql, kl, vl = (t.clone().requires_grad_(True) for t in mine[:3])
                dist.barrier()
                torch.cuda.synchronize()
                ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
                ev[0].record()
                for _ in range(args.time):
                    out = cpar.ring_attention(ql, kl, vl, ctx=cp, comm=comm)
                    out.backward(mine[3])
                    ql.grad = kl.grad = vl.grad = None
                ev[1].record()
                torch.cuda.synchronize()
                t = torch.tensor([ev[0].elapsed_time(ev[1]) / args.time], device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                times[comm] = float(t.item())
        torch.cuda.synchronize()
        names = ("out", "dq", "dk", "dv")
        diffs = {n: float((a - c).abs().max() / (c.abs().max() + 1e-6)) for n, a, c in zip(names, res["p2p"], res["nccl"])}
        if not args.no_check:
            qr, kr, vr = (t.float().to(dev).requires_grad_(True) for t in (q, k, v))
            grp = hq // hkv
            ref = torch.nn.functional.scaled_dot_product_attention(
                qr.transpose(1, 2), kr.repeat_interleave(grp, dim=2).transpose(1, 2),
                vr.repeat_interleave(grp, dim=2).transpose(1, 2), is_causal=True).transpose(1, 2)
            ref.backward(do.float().to(dev))
            refs = [cpar.zigzag_split(t, world, rank) for t in (ref.detach(), qr.grad, kr.grad, vr.grad)]
            for n, a, c in zip(names, res["p2p"], refs):
                diffs[n + "_vs_fp32"] = float((a - c).abs().max() / (c.abs().max() + 1e-6))
        diffs["status"] = native.kernel_status(dev)
        diffs["ms"] = times
        gathered = [None] * world
        dist.all_gather_object(gathered, diffs)
        if rank == 0:
            with open(args.out, "w") as fh:
                json.dump(gathered, fh)


if __name__ == "__main__":
    main()
