"""Worker of the broadcast-load test: rank 0 alone can read the checkpoint directory (the other ranks are given a path
that does not exist); every rank must end up with the same checkpoint through ``broadcast=True``.  Gloo ranks, torchrun."""

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import torch  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ckpt", required=True)
    ap.add_argument("--out", required=True)
    args = ap.parse_args()
    from astrai_b200.parallel import broadcast_state_dict
    from astrai_b200.parallel.setup import setup_parallel
    from astrai_b200.serialization import Checkpoint

    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    with setup_parallel(rank, world, local, "gloo", os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"], "cpu"):
        path = args.ckpt if rank == 0 else args.ckpt + ".not-visible-here"
        ck = Checkpoint.load(path, broadcast=True)
        sd = broadcast_state_dict(ck.state_dict if rank == 0 else None)
        res = {"rank": rank, "epoch": ck.epoch, "consumed": ck.consumed_samples, "keys": sorted(ck.state_dict),
               "sum": float(sum(v.double().sum() for v in ck.state_dict.values())), "extra": sorted(ck.extra),
               "opt_step": ck.extra["optimizer"]["step"], "meta_note": ck.meta.get("note"), "config": ck.config,
               "bsd_sum": float(sum(v.double().sum() for v in sd.values())),
               "dtypes": sorted({str(v.dtype) for v in ck.state_dict.values()})}
        with open(f"{args.out}.{rank}", "w") as fh:
            json.dump(res, fh)


if __name__ == "__main__":
    main()
