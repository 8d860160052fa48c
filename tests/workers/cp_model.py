"""Worker of the multi-GPU sequence-sharded training test: a small bf16 decoder runs one forward + backward on each
rank's zig-zag share of the sequence (context-parallel attention installed), and the result - loss averaged over the
ranks, parameter gradients summed over the ranks - is compared with the same model on the whole sequence on one GPU.
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
    args = ap.parse_args()
    from astrai_b200.config import AutoRegressiveLMConfig
    from astrai_b200.models import AutoRegressiveLM
    from astrai_b200.ops import native
    from astrai_b200.parallel import context_parallel as cpar
    from astrai_b200.parallel.setup import setup_parallel

    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    with setup_parallel(rank, world, local, "nccl", os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"], "cuda"):
        dev = torch.device("cuda", local)
        native.require()
        b, s = 2, 512 * world
        cfg = AutoRegressiveLMConfig(vocab_size=512, hidden_size=256, num_hidden_layers=2, num_attention_heads=4,
                                     num_key_value_heads=2, intermediate_size=512, max_position_embeddings=s,
                                     tie_word_embeddings=False, rms_norm_eps=1e-6, rope_theta=10000.0)
        torch.manual_seed(21)
        model = AutoRegressiveLM(cfg).to(dev).to(torch.bfloat16)
        g = torch.Generator().manual_seed(3)
        ids = torch.randint(0, 512, (b, s), generator=g).to(dev)
        tgt = torch.randint(0, 512, (b, s), generator=g).to(dev)

        def loss_of(logits, targets):
            return torch.nn.functional.cross_entropy(logits.reshape(-1, 512).float(), targets.reshape(-1))

        # whole sequence on this GPU
        loss_full = loss_of(model(ids)["logits"], tgt)
        loss_full.backward()
        ref = {k: p.grad.float().clone() for k, p in model.named_parameters()}
        model.zero_grad()

        cpar.init_context_parallel(cpar.arena_bytes_for(b, s, world, 2, 64), timeout_s=30.0)
        pos = cpar.zigzag_positions(s, world, rank, device=dev).unsqueeze(0).expand(b, -1)
        out = model(cpar.zigzag_split(ids, world, rank), position_ids=pos)
        loss = loss_of(out["logits"], cpar.zigzag_split(tgt, world, rank))
        (loss / world).backward()  # every rank holds 1 / world of the tokens
        worst = 0.0
        for k, p in model.named_parameters():
            gsum = p.grad.float().clone()
            dist.all_reduce(gsum)
            worst = max(worst, float((gsum - ref[k]).abs().max() / (ref[k].abs().max() + 1e-6)))
        lsum = loss.detach().float().clone()
        dist.all_reduce(lsum)
        cpar.set_context(None)
        res = {"loss_full": float(loss_full), "loss_cp": float(lsum / world), "worst_grad": worst, "status": native.kernel_status(dev)}
        gathered = [None] * world
        dist.all_gather_object(gathered, res)
        if rank == 0:
            with open(args.out, "w") as fh:
                json.dump(gathered, fh)


if __name__ == "__main__":
    main()
