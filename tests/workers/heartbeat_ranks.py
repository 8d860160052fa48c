"""Worker of the rank-failure test (CPU, gloo): the ranks all-reduce once per step and beat; ``--victim`` leaves between
steps (orderly ``leave`` or silently, per ``--mode``); the survivors must notice before their next collective, stop
and report.  Launched by torchrun."""

import argparse
import json
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", required=True)
    ap.add_argument("--victim", type=int, default=1)
    ap.add_argument("--mode", choices=["leave", "silent"], default="leave")
    args = ap.parse_args()
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    from astrai_b200.parallel.watchdog import Heartbeat, RankFailure

    hb = Heartbeat(rank, world, timeout_s=1.5, interval_s=0.1).start()
    res = {"rank": rank, "steps": 0, "detected": None, "seconds": None}
    t_gone = None
    try:
        for step in range(1, 200):
            if rank == args.victim and step == 4:  # between steps: nothing of this rank is in flight
                if args.mode == "leave":
                    hb.leave("test")
                hb.stop()
                res["left_at"] = step
                break
            if step == 4:
                t_gone = time.time()
                # the watchdog thread needs a scan (or the timeout) to see it; a live rank keeps beating meanwhile
                for _ in range(3 if args.mode == "leave" else 25):
                    time.sleep(0.1)
                    hb.beat(step - 1)
            hb.check()
            x = torch.ones(4) * rank
            dist.all_reduce(x)
            hb.beat(step)
            res["steps"] = step
    except RankFailure as exc:
        res["detected"] = exc.ranks
        res["seconds"] = time.time() - t_gone if t_gone else None
    hb.stop()
    with open(f"{args.out}.{rank}", "w") as fh:
        json.dump(res, fh)
    os._exit(0)  # no destroy_process_group: the group is missing a member


if __name__ == "__main__":
    main()
