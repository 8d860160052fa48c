"""Worker of the multi-GPU FSDP test: trains a small decoder for a few optimizer steps with the given ``--comm`` and
writes rank 0's losses, gradient norms and a parameter checksum to ``--out`` (JSON).  Launched by torchrun."""

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import torch  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--comm", default="nccl")
    ap.add_argument("--out", required=True)
    ap.add_argument("--steps", type=int, default=4)
    args = ap.parse_args()

    from astrai_b200.config import AutoRegressiveLMConfig
    from astrai_b200.models import AutoRegressiveLM
    from astrai_b200 import ops
    from astrai_b200.optim import FusedAdamW
    from astrai_b200.parallel import ExecutorFactory
    from astrai_b200.parallel.setup import setup_parallel

    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    cfg = AutoRegressiveLMConfig(vocab_size=2048, hidden_size=256, num_hidden_layers=3, rms_norm_eps=1e-6,
                                 intermediate_size=512, tie_word_embeddings=True, max_position_embeddings=256,
                                 rope_theta=10000.0, num_attention_heads=4, num_key_value_heads=2)
    accum = 2
    with setup_parallel(rank, world, local, "nccl", os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"], "cuda"):
        dev = torch.device("cuda", local)

        def model_fn():
            torch.manual_seed(7)
            return AutoRegressiveLM(cfg).to(dev, torch.bfloat16)

        ex = ExecutorFactory.create("fsdp", grad_accum_steps=accum, comm=args.comm, comm_timeout_s=30.0)
        model, opt, _ = ex.prepare(model_fn, lambda m: FusedAdamW(m.parameters(), lr=1e-3, weight_decay=0.1))
        model.train()
        g = torch.Generator().manual_seed(100 + rank)
        losses, norms = [], []
        for step in range(args.steps):
            for micro in range(accum):
                ids = torch.randint(0, cfg.vocab_size, (2, 129), generator=g).to(dev)
                with ex.accumulate(model):
                    with ops.assume_loss_grad(1.0 / accum):
                        out = model(ids[:, :-1], return_logits=False)
                        loss = ops.linear_cross_entropy(out["hidden_states"], model.lm_head.weight, ids[:, 1:], 0.0)
                    ex.backward(loss, torch.full_like(loss, 1.0 / accum))
                    if ex.sync_gradients:
                        norms.append(ex.clip_grad_norm(model, 1.0))
                        opt.step()
                        opt.zero_grad()
            losses.append(float(loss.item()))
        sd = ex.unwrap_model(model)
        torch.cuda.synchronize()
        from astrai_b200.ops import native

        status = native.kernel_status(dev)
        if rank == 0:
            checksum = float(sum(v.float().abs().sum().item() for v in sd.values()))
            with open(args.out, "w") as fh:
                json.dump({"losses": losses, "norms": norms, "checksum": checksum, "status": status}, fh)


if __name__ == "__main__":
    main()
