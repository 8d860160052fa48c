"""Worker of the pipeline-parallel test (CPU, gloo): every rank builds the same tiny model, the group runs one 1F1B
step over it, and each stage compares its loss / gradients with a plain forward + backward of the whole model."""

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
    ap.add_argument("--micro", type=int, default=4)
    ap.add_argument("--moe", action="store_true")
    ap.add_argument("--sft", action="store_true", help="packed documents with a loss mask: the loss is a mean over the trained tokens")
    args = ap.parse_args()
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    from astrai_b200.config import AutoRegressiveLMConfig
    from astrai_b200.models.lm import AutoRegressiveLM
    from astrai_b200.parallel.pipeline import PipelineParallel

    extra = dict(ffn_type="moe", n_routed_experts=4, n_activated_experts=2, moe_intermediate_size=16, n_shared_experts=1) if args.moe else {}
    cfg = AutoRegressiveLMConfig(vocab_size=97, hidden_size=32, num_hidden_layers=5, num_attention_heads=4, num_key_value_heads=2,
                                 intermediate_size=64, max_position_embeddings=64, tie_word_embeddings=False, **extra)
    torch.manual_seed(11)
    model = AutoRegressiveLM(cfg)
    ref = AutoRegressiveLM(cfg)
    ref.load_state_dict(model.state_dict())
    ids = torch.randint(0, 97, (8, 16))
    targets = torch.randint(0, 97, (8, 16))
    coef = 0.01 if args.moe else 0.0

    kwargs = weights = None
    if args.sft:
        from astrai_b200.trainer.strategy import doc_attention

        # rows of two or three packed documents of different lengths; about a third of the tokens are trained, unevenly
        g = torch.Generator().manual_seed(5)
        cuts = [sorted(torch.randperm(15, generator=g)[: 1 + r % 2].add(1).tolist()) for r in range(8)]
        pos = torch.stack([torch.cat([torch.arange(b - a) for a, b in zip([0] + c, c + [16])]) for c in cuts])
        keep = torch.rand(8, 16, generator=g) < torch.linspace(0.1, 0.7, 8)[:, None]
        targets = targets.masked_fill(~keep, -100)
        # the whole batch's mean over its trained tokens, accumulated piece by piece (the router loss is not a sum over
        # tokens, so the whole model must see the same pieces as the stages for its gradients to be comparable)
        n_trained = int(keep.sum())
        total = 0.0
        for xi, ti, pi in zip(ids.chunk(args.micro), targets.chunk(args.micro), pos.chunk(args.micro)):
            out = ref(xi, input_mask=doc_attention(pi), position_ids=pi)
            loss = torch.nn.functional.cross_entropy(out["logits"].reshape(-1, 97).float(), ti.reshape(-1), ignore_index=-100,
                                                     reduction="sum") / n_trained
            total += loss.item()
            if args.moe:
                loss = loss + coef * out["aux_loss"] / args.micro
            loss.backward()
        if not args.moe:  # and in one piece: the same number
            whole = ref(ids, input_mask=doc_attention(pos), position_ids=pos)["logits"]
            one = torch.nn.functional.cross_entropy(whole.reshape(-1, 97).float(), targets.reshape(-1), ignore_index=-100)
            assert abs(one.item() - total) < 1e-5, (one.item(), total)
        kwargs = [{"position_ids": p, "attention": doc_attention(p)} for p in pos.chunk(args.micro)]
        counts = keep.reshape(args.micro, -1).sum(1).double()
        weights = (counts / counts.sum()).tolist()
    else:
        # whole model, same micro-batching (the loss is a mean of per-micro-batch means)
        total = 0.0
        for xi, ti in zip(ids.chunk(args.micro), targets.chunk(args.micro)):
            out = ref(xi)
            loss = torch.nn.functional.cross_entropy(out["logits"].reshape(-1, 97).float(), ti.reshape(-1))
            total += loss.item() / args.micro
            if args.moe:
                loss = loss + coef * out["aux_loss"]  # the stages' shares add up to the model's mean over its layers
            (loss / args.micro).backward()

    def loss_fn(logits, t):
        return torch.nn.functional.cross_entropy(logits.reshape(-1, logits.size(-1)).float(), t.reshape(-1), ignore_index=-100)

    pp = PipelineParallel(model, aux_loss_coef=coef, loss_fn=loss_fn)
    loss = pp.train_step(ids if rank == 0 else None, targets if rank == world - 1 else None, args.micro, micro_shape=(8 // args.micro, 16),
                         micro_kwargs=kwargs, weights=weights)
    ref_grads = dict(ref.named_parameters())
    worst = 0.0
    for key in pp.stage.owned_keys(model):
        g = dict(model.named_parameters())[key].grad
        rg = ref_grads[key].grad
        assert g is not None, key
        worst = max(worst, float((g - rg).abs().max() / (rg.abs().max() + 1e-8)))
    not_mine = [k for k, p in model.named_parameters() if p.grad is not None and k not in set(pp.stage.owned_keys(model))]
    res = {"rank": rank, "worst": worst, "loss": None if loss is None else float(loss), "ref_loss": total, "stray": not_mine,
           "n_keys": len(pp.stage.owned_keys(model))}
    gathered = [None] * world
    dist.all_gather_object(gathered, res)
    if rank == 0:
        with open(args.out, "w") as fh:
            json.dump(gathered, fh)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
