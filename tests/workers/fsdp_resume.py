"""Worker of the sharded save / resume test: trains a small decoder under the flat FSDP executor, once without
interruption and once with a checkpoint (model + gathered optimizer state) written and re-loaded half way by freshly
built objects on every rank, and writes both runs' losses and parameter checksums to ``--out``.  Runs on gloo ranks
(CPU) or NCCL ranks (GPU); launched by torchrun."""

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import torch  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", required=True)
    ap.add_argument("--ckpt", required=True)
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--comm", default="nccl")
    ap.add_argument("--untied", action="store_true")
    args = ap.parse_args()

    from astrai_b200.config import AutoRegressiveLMConfig
    from astrai_b200.models import AutoRegressiveLM
    from astrai_b200 import ops
    from astrai_b200.optim import FusedAdamW
    from astrai_b200.parallel import ExecutorFactory
    from astrai_b200.parallel.setup import setup_parallel
    from astrai_b200.serialization import Checkpoint

    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    cuda = args.device == "cuda"
    cfg = AutoRegressiveLMConfig(vocab_size=512, hidden_size=128, num_hidden_layers=2, rms_norm_eps=1e-6,
                                 intermediate_size=256, tie_word_embeddings=not args.untied, max_position_embeddings=128,
                                 rope_theta=10000.0, num_attention_heads=2, num_key_value_heads=1)
    accum, total, half = 2, 4, 2
    with setup_parallel(rank, world, local, "nccl" if cuda else "gloo", os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"],
                        "cuda" if cuda else "cpu"):
        dev = torch.device("cuda", local) if cuda else torch.device("cpu")

        def build(state=None, opt_state=None):
            def model_fn():
                torch.manual_seed(7)
                return AutoRegressiveLM(cfg).to(dev, torch.bfloat16)

            def before_wrap(m):
                if state is not None:
                    m.load_state_dict(state)
                return m

            kw = dict(comm=args.comm, comm_timeout_s=30.0) if cuda else dict(impl="flat")
            ex = ExecutorFactory.create("fsdp", grad_accum_steps=accum, **kw)
            model, opt, _ = ex.prepare(model_fn, lambda m: FusedAdamW(m.parameters(), lr=1e-2, weight_decay=0.1),
                                       before_wrap=before_wrap)
            if opt_state is not None:
                opt.load_state_dict(opt_state)
            model.train()
            return ex, model, opt

        def batch(step, micro):
            g = torch.Generator().manual_seed(1000 * step + 10 * micro + rank)
            return torch.randint(0, cfg.vocab_size, (2, 65), generator=g).to(dev)

        def run(ex, model, opt, steps):
            losses = []
            for step in steps:
                for micro in range(accum):
                    ids = batch(step, micro)
                    with ex.accumulate(model):
                        if cuda:
                            with ops.assume_loss_grad(1.0 / accum):
                                out = model(ids[:, :-1], return_logits=False)
                                ex.before_param_use(model.lm_head.weight)
                                loss = ops.linear_cross_entropy(out["hidden_states"], model.lm_head.weight, ids[:, 1:], 0.0)
                            ex.backward(loss, torch.full_like(loss, 1.0 / accum))
                        else:
                            logits = model(ids[:, :-1])["logits"]
                            loss = ops.cross_entropy(logits, ids[:, 1:])
                            ex.backward(loss / accum)
                        if ex.sync_gradients:
                            ex.clip_grad_norm(model, 1.0)
                            opt.step()
                            opt.zero_grad()
                losses.append(float(loss.item()))
            return losses

        def checksum(ex, model):
            sd = ex.unwrap_model(model)
            return float(sum(v.float().abs().sum().item() for v in sd.values())) if sd is not None else None

        # (a) uninterrupted
        ex, model, opt = build()
        a_losses = run(ex, model, opt, range(total))
        a_sum = checksum(ex, model)
        # (b) first half, save, rebuild everything, load, second half
        ex, model, opt = build()
        b_losses = run(ex, model, opt, range(half))
        extra = {"optimizer": opt.state_dict()}  # collective: every rank's shard is gathered, rank 0 keeps the whole
        with ex.checkpoint_context(model) as sd:
            if sd is not None:
                Checkpoint(state_dict=sd, epoch=0, consumed_samples=0, extra=extra, config=cfg.to_dict()).save(args.ckpt)
        del ex, model, opt
        ck = Checkpoint.load(args.ckpt)
        layout = ck.extra["optimizer"]["flat_layout"]
        ex, model, opt = build(ck.state_dict, ck.extra["optimizer"])
        b_losses += run(ex, model, opt, range(half, total))
        b_sum = checksum(ex, model)
        if cuda:
            torch.cuda.synchronize()
        if rank == 0:
            with open(args.out, "w") as fh:
                json.dump({"a": a_losses, "b": b_losses, "a_sum": a_sum, "b_sum": b_sum, "layout": layout}, fh)


if __name__ == "__main__":
    main()
