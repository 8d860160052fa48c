"""Worker of the full-shard residency test: the same small decoder is trained under the flat FSDP executor twice, with the
replicated placement and with ``reshard=True`` (parameters and gradients whole only while their unit computes), on the
same micro-batches; both runs' losses, gradient norms and final weights, and the residency bookkeeping of the second run,
go to ``--out``.  Runs on gloo ranks (CPU) or NCCL ranks (GPU); launched by torchrun."""

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import torch  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", required=True)
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--untied", action="store_true")
    ap.add_argument("--layers", type=int, default=3)
    args = ap.parse_args()

    from astrai_b200 import ops
    from astrai_b200.config import AutoRegressiveLMConfig
    from astrai_b200.models import AutoRegressiveLM
    from astrai_b200.optim import FusedAdamW
    from astrai_b200.parallel import ExecutorFactory
    from astrai_b200.parallel.setup import setup_parallel

    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    cuda = args.device == "cuda"
    dtype = torch.bfloat16 if cuda else torch.float32
    cfg = AutoRegressiveLMConfig(vocab_size=512, hidden_size=128, num_hidden_layers=args.layers, rms_norm_eps=1e-6,
                                 intermediate_size=256, tie_word_embeddings=not args.untied, max_position_embeddings=128,
                                 rope_theta=10000.0, num_attention_heads=2, num_key_value_heads=1)
    accum, steps = 2, 3
    with setup_parallel(rank, world, local, "nccl" if cuda else "gloo", os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"],
                        "cuda" if cuda else "cpu"):
        dev = torch.device("cuda", local) if cuda else torch.device("cpu")

        def build(reshard):
            def model_fn():
                torch.manual_seed(7)
                return AutoRegressiveLM(cfg).to(dev, dtype)

            ex = ExecutorFactory.create("fsdp", grad_accum_steps=accum, impl="flat", comm="nccl", reshard=reshard)
            model, opt, _ = ex.prepare(model_fn, lambda m: FusedAdamW(m.parameters(), lr=1e-3, weight_decay=0.1))
            model.train()
            return ex, model, opt

        def batch(step, micro):
            g = torch.Generator().manual_seed(1000 * step + 10 * micro + rank)
            return torch.randint(0, cfg.vocab_size, (2, 65), generator=g).to(dev)

        def run(reshard):
            ex, model, opt = build(reshard)
            rs = ex._rs
            info = {"at_rest_after_prepare": rs.resident_bytes() if rs is not None else None}
            losses, norms, mid = [], [], []
            for step in range(steps):
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
                        if rs is not None:
                            mid.append(rs.resident_bytes())  # between micro-batches: everything released again
                        if ex.sync_gradients:
                            norms.append(ex.clip_grad_norm(model, 1.0))
                            opt.step()
                            opt.zero_grad()
                losses.append(float(loss.item()))
            with torch.no_grad():  # an evaluation pass gathers and releases as well
                ids = batch(99, 0)
                eval_loss = float(ops.cross_entropy(model(ids[:, :-1])["logits"].float(), ids[:, 1:]).item())
            peak = rs.peak_resident_params if rs is not None else None  # before the save, which gathers every unit
            sd = ex.unwrap_model(model)
            if rs is not None:
                info.update(between_micro_batches=max(mid), peak_units=peak, units=len(ex.engine.units),
                            at_rest_after_save=rs.resident_bytes(),
                            whole_bytes=sum(u.numel * (u.param_buf.element_size() + 4) for u in ex.engine.units))
            if cuda:
                torch.cuda.synchronize()
            return losses, norms, eval_loss, sd, info

        a_losses, a_norms, a_eval, a_sd, _ = run(False)
        b_losses, b_norms, b_eval, b_sd, info = run(True)
        if rank == 0:
            diff = max(float((a_sd[k].float() - b_sd[k].float()).abs().max()) for k in a_sd)
            with open(args.out, "w") as fh:
                json.dump({"a": a_losses, "b": b_losses, "a_norms": a_norms, "b_norms": b_norms, "a_eval": a_eval, "b_eval": b_eval,
                           "max_weight_diff": diff, "keys": sorted(a_sd) == sorted(b_sd), "info": info}, fh)


if __name__ == "__main__":
    main()
