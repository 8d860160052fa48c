"""Worker of the model-parallel trainer tests: runs the real ``Trainer`` for a few optimizer steps in one of the modes
``tp | cp | ep | pp`` (``--mode``, ``--size``) and writes the per-step losses, the gradient norms and the final (gathered,
unsharded) state dict's checksums to ``--out``.  With ``--mode none`` and one process it produces the single-process
reference over the same global batches.  Runs on gloo ranks (CPU) or NCCL ranks (GPU); launched by torchrun."""

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import torch  # noqa: E402


class Tokens(torch.utils.data.Dataset):
    def __init__(self, n, seq, vocab, seed=0):
        g = torch.Generator().manual_seed(seed)
        self.data = torch.randint(1, vocab, (n, seq + 1), generator=g)

    def __len__(self):
        return self.data.shape[0]

    def __getitem__(self, i):
        row = self.data[i]
        return {"input_ids": row[:-1], "target_ids": row[1:]}


class PackedChats(Tokens):
    """Rows of two or three packed documents (position ids restart) with an uneven share of trained tokens per row."""

    def __getitem__(self, i):
        row = self.data[i]
        seq = row.numel() - 1
        g = torch.Generator().manual_seed(1000 + i)
        cuts = sorted(torch.randperm(seq - 1, generator=g)[: 1 + i % 2].add(1).tolist())
        pos = torch.cat([torch.arange(b - a) for a, b in zip([0] + cuts, cuts + [seq])])
        keep = torch.rand(seq, generator=g) < (0.15 + 0.2 * (i % 4))
        keep[0] = True
        return {"input_ids": row[:-1], "target_ids": row[1:], "position_ids": pos, "loss_mask": keep}


class Pairs(torch.utils.data.Dataset):
    """Preference pairs with a shared masked prompt and right padding of uneven length (token id 0)."""

    def __init__(self, n, seq, vocab, seed=0):
        g = torch.Generator().manual_seed(seed)
        self.chosen = torch.randint(3, vocab, (n, seq), generator=g)
        self.rejected = torch.randint(3, vocab, (n, seq), generator=g)
        self.rejected[:, :4] = self.chosen[:, :4]
        self.cmask = torch.zeros(n, seq, dtype=torch.bool)
        self.rmask = torch.zeros(n, seq, dtype=torch.bool)
        for i in range(n):
            lc, lr = seq - (i % 5), seq - ((i + 2) % 7)
            self.chosen[i, lc:], self.rejected[i, lr:] = 0, 0
            self.cmask[i, 4:lc], self.rmask[i, 4:lr] = True, True

    def __len__(self):
        return self.chosen.shape[0]

    def __getitem__(self, i):
        return {"chosen": self.chosen[i], "rejected": self.rejected[i], "chosen_mask": self.cmask[i], "rejected_mask": self.rmask[i]}


class Groups(torch.utils.data.Dataset):
    """Prompts (left-padded) with three scored responses each (right-padded)."""

    def __init__(self, n, seq, vocab, seed=0):
        g = torch.Generator().manual_seed(seed)
        plen, rlen = seq // 2, seq // 2 - 1  # an odd total length on purpose
        self.prompts = torch.randint(3, vocab, (n, plen), generator=g)
        self.responses = torch.randint(3, vocab, (n, 3, rlen), generator=g)
        self.masks = torch.ones(n, 3, rlen, dtype=torch.bool)
        self.rewards = torch.rand(n, 3, generator=g)
        for i in range(n):
            self.prompts[i, : i % 3] = 0
            cut = rlen - (i % 4)
            self.responses[i, 1, cut:] = 0
            self.masks[i, 1, cut:] = False

    def __len__(self):
        return self.prompts.shape[0]

    def __getitem__(self, i):
        return {"prompts": self.prompts[i], "responses": self.responses[i], "masks": self.masks[i], "rewards": self.rewards[i]}


class Record:
    def __init__(self):
        self.losses, self.norms, self.val = [], [], []

    def on_optimizer_step(self, context):
        import torch.distributed as dist

        loss = torch.tensor([float(context.loss)], dtype=torch.float64, device=context.strategy.device)
        if dist.is_initialized():  # every rank reports the mean over its own tokens: the job's loss is their mean
            dist.all_reduce(loss)
            loss /= dist.get_world_size()
        self.losses.append(float(loss))
        self.norms.append(float(context.grad_norm) if context.grad_norm is not None else None)

    def on_train_end(self, context):
        if getattr(context, "val_dataloader", None) is not None:
            from astrai_b200.trainer.train_callback import MetricCallback

            self.val.append(MetricCallback(context.config.ckpt_dir, 10**6, ["loss"])._validate(context))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", required=True)
    ap.add_argument("--ckpt", required=True)
    ap.add_argument("--mode", default="tp")
    ap.add_argument("--size", type=int, default=0)
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--comm", default="nccl")
    ap.add_argument("--moe", action="store_true")
    ap.add_argument("--seq", type=int, default=32)
    ap.add_argument("--hidden", type=int, default=32)
    ap.add_argument("--bpd", type=int, default=2)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--dtype", default="float32")
    ap.add_argument("--lr", type=float, default=1e-2)
    ap.add_argument("--chunks", type=int, default=0)
    ap.add_argument("--layers", type=int, default=2)
    ap.add_argument("--strategy", default="seq", choices=["seq", "sft", "dpo", "grpo"])
    ap.add_argument("--val", action="store_true", help="hold a quarter of the data out and report its loss after training")
    ap.add_argument("--label_smoothing", type=float, default=0.0)
    args = ap.parse_args()

    from astrai_b200.config import AutoRegressiveLMConfig, TrainConfig
    from astrai_b200.models import AutoRegressiveLM
    from astrai_b200.optim import FusedAdamW
    from astrai_b200.trainer import Trainer

    world = int(os.environ.get("WORLD_SIZE", "1"))
    cuda = args.device == "cuda"
    dtype = getattr(torch, args.dtype)
    extra = dict(ffn_type="moe", n_routed_experts=4, n_shared_experts=1, n_activated_experts=2,
                 moe_intermediate_size=args.hidden * 2) if args.moe else {}
    cfg = AutoRegressiveLMConfig(vocab_size=256, hidden_size=args.hidden, num_hidden_layers=args.layers, rms_norm_eps=1e-6,
                                 intermediate_size=args.hidden * 2, tie_word_embeddings=False,
                                 max_position_embeddings=args.seq, rope_theta=10000.0,
                                 num_attention_heads=max(args.hidden // (128 if cuda else 8), 2),
                                 num_key_value_heads=2, **extra)

    def model_fn():
        torch.manual_seed(11)
        return AutoRegressiveLM(cfg).to(dtype)

    accum = 2
    # the same global batch in every run: ranks of one tp / cp block share their samples, so the per-device batch of
    # those modes is the single-process one; ep ranks (and plain data parallelism) split it
    from astrai_b200.parallel.mesh import data_parallel_size
    dw = data_parallel_size(args.mode, world, args.size, args.size, args.size, args.size)
    global_batch = args.bpd * 2
    bpd = global_batch // dw
    n = global_batch * accum * args.steps
    data_cls = {"sft": PackedChats, "dpo": Pairs, "grpo": Groups}.get(args.strategy, Tokens)
    objective = {"dpo": {"beta": 0.5}, "grpo": {"group_size": 3, "clip_eps": 0.2, "kl_coef": 0.05}}.get(args.strategy, {})
    if args.val:
        n = n * 4 // 3  # the held-out quarter comes off the end
    exkw = {"comm": args.comm} if args.mode in ("tp", "cp", "ep") else {}
    if args.mode == "pp" and args.chunks:
        exkw["chunks"] = args.chunks
    if args.mode == "cp":  # the gradient / parameter transport and the attention transport are chosen together here
        exkw["attn_comm"] = args.comm
        exkw["max_tokens_per_rank"] = bpd * args.seq // max(world // max(dw, 1), 1) * 2
    if args.mode == "ep":
        exkw["tokens_per_rank"] = bpd * args.seq
    tc = TrainConfig(model_fn=model_fn, strategy=args.strategy, dataset=data_cls(n, args.seq, 256),
                     val_split=0.25 if args.val else None, val_step=10**6,
                     strategy_kwargs={"label_smoothing": args.label_smoothing} if args.label_smoothing else objective,
                     optimizer_fn=lambda m: FusedAdamW(m.parameters(), lr=args.lr, weight_decay=0.0),
                     batch_per_device=bpd, grad_accum_steps=accum, ckpt_dir=args.ckpt, ckpt_interval=10**6,
                     device_type="cuda" if cuda else "cpu", backend="nccl" if cuda else "gloo", nprocs=world,
                     parallel_mode=args.mode, tp_size=args.size or 1, cp_size=args.size or 1, ep_size=args.size or 1, pp_size=args.size or 1,
                     executor_kwargs=exkw, max_grad_norm=1.0, moe_aux_loss_coef=0.0,
                     master_addr=os.environ.get("MASTER_ADDR", "127.0.0.1"), master_port=os.environ.get("MASTER_PORT", "29500"))
    rec = Record()
    trainer = Trainer(tc, callbacks=[rec])
    trainer.callbacks = [cb for cb in trainer.callbacks if type(cb).__name__ not in ("ProgressBarCallback", "MetricCallback")]
    # deterministic order: the sampler must not shuffle differently between the runs that are compared
    import astrai_b200.trainer.train_context as tcx
    orig = tcx.RDSampler

    def fixed(ds, **kw):
        kw["shuffle"] = False
        return orig(ds, **kw)

    tcx.RDSampler = fixed
    trainer.train()
    if int(os.environ.get("RANK", "0")) == 0:
        from astrai_b200.serialization import Checkpoint
        from pathlib import Path

        last = sorted(Path(args.ckpt).glob("epoch_*"), key=lambda p: p.stat().st_mtime)[-1]
        ck = Checkpoint.load(last)
        sd = ck.state_dict
        opt_state = ck.extra.get("optimizer")
        stages = len(opt_state["pipeline_stages"]) if isinstance(opt_state, dict) and "pipeline_stages" in opt_state else 0
        sums = {k: float(v.float().abs().sum()) for k, v in sd.items()}
        shapes = {k: list(v.shape) for k, v in sd.items()}
        with open(args.out, "w") as fh:
            json.dump({"losses": rec.losses, "norms": rec.norms, "val": rec.val, "sums": sums, "shapes": shapes, "optimizer_stages": stages}, fh)


if __name__ == "__main__":
    main()
