"""Worker of the multi-GPU tensor-parallel test: a sequence-sharded SwiGLU MLP (column-parallel gate/up, row-parallel
down) run forward + backward with fused peer-memory kernels and with NCCL collectives around the plain GEMM; rank 0
writes the largest differences of outputs and gradients to ``--out``.  Launched by torchrun."""

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
    args = ap.parse_args()
    from astrai_b200.ops import native
    from astrai_b200.parallel import tensor_parallel as tp
    from astrai_b200.parallel.setup import setup_parallel

    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    with setup_parallel(rank, world, local, "nccl", os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"], "cuda"):
        dev = torch.device("cuda", local)
        native.require()
        tp.init_tensor_parallel(arena_bytes=256 << 20, timeout_s=30.0)
        dim, hidden, tokens = 512, 1536, 256 * world
        torch.manual_seed(3)
        gate = (torch.randn(hidden, dim) * 0.03).bfloat16().to(dev)
        up = (torch.randn(hidden, dim) * 0.03).bfloat16().to(dev)
        down = (torch.randn(dim, hidden) * 0.03).bfloat16().to(dev)
        x_all = torch.randn(tokens, dim).bfloat16().to(dev)
        gy_all = torch.randn(tokens, dim).bfloat16().to(dev)
        sl = slice(rank * tokens // world, (rank + 1) * tokens // world)
        res = {}
        for comm in ("nccl", "p2p"):
            mlp = tp.TensorParallelMLP(dim, hidden, world, rank, comm=comm, dtype=torch.bfloat16, device=dev)
            with torch.no_grad():
                mlp.gate_up.weight.copy_(tp.TensorParallelMLP.shard_gate_up(gate, up, world, rank))
                mlp.down.weight.copy_(tp.RowParallelLinear.shard(down, world, rank))
            outs = []
            for _ in range(3):  # several calls: buffer parity and epochs advance
                x = x_all[sl].clone().requires_grad_(True)
                y = mlp(x)
                y.backward(gy_all[sl])
                outs.append((y.detach().float(), x.grad.float(), mlp.gate_up.weight.grad.float().clone(), mlp.down.weight.grad.float().clone()))
                mlp.zero_grad()
            res[comm] = outs[-1]
        torch.cuda.synchronize()
        names = ("y", "dx", "d_gate_up", "d_down")
        diffs = {n: float((a - b).abs().max() / (b.abs().max() + 1e-6)) for n, a, b in zip(names, res["p2p"], res["nccl"])}
        # reference in fp32 on rank 0's slice
        h = torch.nn.functional.silu(x_all.float() @ gate.float().t()) * (x_all.float() @ up.float().t())
        ref = (h @ down.float().t())[sl]
        diffs["y_vs_fp32"] = float((res["p2p"][0] - ref).abs().max() / (ref.abs().max() + 1e-6))
        diffs["status"] = native.kernel_status(dev)
        gathered = [None] * world
        dist.all_gather_object(gathered, diffs)
        if rank == 0:
            with open(args.out, "w") as fh:
                json.dump(gathered, fh)


if __name__ == "__main__":
    main()
