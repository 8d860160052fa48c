"""Where one micro-batch of the 1B training step spends its GPU time.

    python -m astrai_b200.utils.step_budget [--layers 24] [--micro 2] [--out budget.md]

Builds the benchmark model (24 layers, d 2048, 16q / 4kv heads, FFN 5632, vocab 32000, tied; batch 4 x 2048 tokens),
runs forward + backward of the ``seq`` objective on the flat single-GPU runtime exactly as the trainer does, and prints

* the CUDA-event time of a micro-batch measured WITHOUT any profiler (the number to trust for the total), and
* a per-kernel table from ``torch.profiler`` (CUPTI kernel durations summed per kernel name over the profiled
  micro-batches, divided by their count): launches, microseconds and share of the kernel-time sum.

The table is a budget - it says which kernels to work on - not a benchmark: kernel durations under CUPTI are slightly
longer than in a free run and their sum ignores gaps and overlap.  The reference has no such tool (its only timer is a
DEBUG-level CUDA-event pair around serving forwards, ``astrai/inference/runtime/executor.py:24-45``).
"""

from __future__ import annotations

import argparse
import collections
import sys

import torch


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=24)
    ap.add_argument("--micro", type=int, default=2, help="micro-batches under the profiler")
    ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--out", default=None)
    ap.add_argument("--top", type=int, default=40)
    args = ap.parse_args(argv)

    from astrai_b200 import ops
    from astrai_b200.config import AutoRegressiveLMConfig
    from astrai_b200.models import AutoRegressiveLM
    from astrai_b200.ops import native
    from astrai_b200.parallel import ExecutorFactory

    native.require()
    dev = torch.device("cuda", 0)
    cfg = AutoRegressiveLMConfig(vocab_size=32000, hidden_size=2048, num_hidden_layers=args.layers, rms_norm_eps=1e-6,
                                 intermediate_size=5632, tie_word_embeddings=True, max_position_embeddings=args.seq,
                                 rope_theta=10000.0, num_attention_heads=16, num_key_value_heads=4)

    def model_fn():
        torch.manual_seed(0)
        return AutoRegressiveLM(cfg).to(dev, torch.bfloat16)

    ex = ExecutorFactory.create("none", grad_accum_steps=10**9)  # never closes a window: forward + backward only
    model, _, _ = ex.prepare(model_fn)
    model.train()
    g = torch.Generator().manual_seed(1)

    def micro():
        ids = torch.randint(0, cfg.vocab_size, (args.batch, args.seq + 1), generator=g).to(dev)
        with ex.accumulate(model), ops.assume_loss_grad(1.0 / 8):
            out = model(ids[:, :-1], return_logits=False)
            loss = ops.linear_cross_entropy(out["hidden_states"], model.lm_head.weight, ids[:, 1:], 0.05)
        ex.backward(loss, torch.full_like(loss, 1.0 / 8))
        return loss

    for _ in range(3):
        micro()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    n_free = 4
    e0.record()
    for _ in range(n_free):
        micro()
    e1.record()
    torch.cuda.synchronize()
    free_ms = e0.elapsed_time(e1) / n_free

    from torch.profiler import ProfilerActivity, profile

    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(args.micro):
            micro()
        torch.cuda.synchronize()
    per = collections.defaultdict(lambda: [0, 0.0])
    for evt in prof.events():
        if evt.device_type == torch.autograd.DeviceType.CUDA and evt.device_time_total > 0:
            name = evt.name.replace("(anonymous namespace)::", "").split("(")[0]
            per[name][0] += 1
            per[name][1] += evt.device_time_total
    rows = sorted(((n, c / args.micro, t / args.micro) for n, (c, t) in per.items()), key=lambda r: -r[2])
    total = sum(r[2] for r in rows)
    tokens = args.batch * args.seq
    lines = [
        f"micro-batch of {tokens} tokens, {args.layers} layers, forward + backward (no optimizer step)",
        f"free-running time (CUDA events, no profiler, mean of {n_free}): {free_ms:.2f} ms  ->  {tokens / free_ms * 1e3:,.0f} tok/s",
        f"sum of kernel durations under torch.profiler: {total / 1e3:.2f} ms over {sum(r[1] for r in rows):.0f} launches",
        "",
        "| kernel | launches / micro-batch | us / micro-batch | share |",
        "|---|---|---|---|",
    ]
    for name, count, us in rows[: args.top]:
        lines.append(f"| `{name[:90]}` | {count:.0f} | {us:,.0f} | {100 * us / total:.1f} % |")
    rest = rows[args.top:]
    if rest:
        lines.append(f"| ({len(rest)} more kernels) | {sum(r[1] for r in rest):.0f} | {sum(r[2] for r in rest):,.0f} | "
                     f"{100 * sum(r[2] for r in rest) / total:.1f} % |")
    text = "\n".join(lines)
    print(text)
    if args.out:
        with open(args.out, "w") as fh:
            fh.write(text + "\n")
    return 0


if __name__ == "__main__":
    sys.exit(main())
