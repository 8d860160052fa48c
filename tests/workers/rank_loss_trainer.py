"""Worker of the emergency-save test (CPU, gloo): three ranks train through the real ``Trainer`` with the heartbeat
callback; ``--victim`` exits between two optimizer steps without a word.  The survivors must notice on the host, write
an emergency checkpoint without any collective and return within a bound.  Launched by torchrun."""

import argparse
import json
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402


class VictimExits:
    """Callback: the victim rank leaves the job at the start of a micro-batch, with nothing of its own in flight."""

    def __init__(self, victim: int, at_step: int, marker: str):
        self.victim, self.at_step, self.marker = victim, at_step, marker

    def on_batch_begin(self, context):
        if context.rank == self.victim and context.optimizer_step >= self.at_step:
            with open(self.marker, "w") as fh:
                fh.write(str(time.time()))
            os._exit(0)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", required=True)
    ap.add_argument("--ckpt", required=True)
    ap.add_argument("--mode", default="fsdp")
    ap.add_argument("--victim", type=int, default=1)
    args = ap.parse_args()
    from helpers import RandomTokens, tiny_config

    from astrai_b200.config import TrainConfig
    from astrai_b200.models import AutoRegressiveLM
    from astrai_b200.optim import FusedAdamW
    from astrai_b200.parallel.watchdog import RankFailure
    from astrai_b200.trainer import Trainer

    rank = int(os.environ["RANK"])

    def model_fn():
        torch.manual_seed(0)
        return AutoRegressiveLM(tiny_config(tie_word_embeddings=True))

    cfg = TrainConfig(model_fn=model_fn, strategy="seq", dataset=RandomTokens(600, 12),
                      optimizer_fn=lambda m: FusedAdamW(m.parameters(), lr=1e-2), batch_per_device=2, grad_accum_steps=2,
                      ckpt_dir=args.ckpt, ckpt_interval=10**6, device_type="cpu", backend="gloo", nprocs=3,
                      parallel_mode=args.mode, executor_kwargs={"impl": "flat"}, heartbeat_timeout_s=1.5,
                      heartbeat_interval_s=0.1, master_addr=os.environ["MASTER_ADDR"], master_port=os.environ["MASTER_PORT"])
    marker = args.out + ".gone"
    trainer = Trainer(cfg, callbacks=[VictimExits(args.victim, 3, marker)])
    trainer.callbacks = [cb for cb in trainer.callbacks if type(cb).__name__ not in ("ProgressBarCallback",)]
    res = {"rank": rank, "failure": None}
    try:
        trainer.train()
    except RankFailure as exc:
        res["failure"] = exc.ranks
    res["returned_at"] = time.time()
    with open(f"{args.out}.{rank}", "w") as fh:
        json.dump(res, fh)
    os._exit(0)  # the process group is missing a member: skip its teardown


if __name__ == "__main__":
    main()
