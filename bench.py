"""Headline benchmark: 1B-class dense decoder pre-training, FSDP, bf16, synthetic packed tokens.

    python bench.py --gpus N --steps K --warmup W [--impl ours|reference] [--config fsdp1b|tp8b|cp8b|ep_moe] [--comm p2p|nccl]

``--config`` selects one of the other training configurations (8B dense with tensor parallelism at seq 8192 / global
batch 8, 8B dense with context parallelism at seq 65 536 / batch 1, MoE + MLA with expert parallelism at seq 4096 /
batch 2 per GPU); ``--comm nccl`` runs the same configuration on library collectives, which is the comparison arm of
those three (the reference cannot run them).  Without ``--config`` the run is the headline described below.

Model / recipe: 24 layers, d_model 2048, 16 query / 4 KV heads (head_dim 128), SwiGLU FFN 5632, vocab 32000, tied
embeddings, RoPE; seq 2048, batch_per_device 4, grad_accum 8 (one "step" = one optimizer step = 65 536 tokens per GPU),
AdamW (lr 1e-4, wd 0.1), label smoothing 0.05, gradient clipping at 1.0.  Weak scaling: per-GPU work is fixed.

Two measurements per run, both over exactly K optimizer steps after W warm-up steps, bracketed by barrier +
``torch.cuda.synchronize()``, timed with CUDA events, max over ranks:
  * ``value``   - the training step driven directly with token batches already resident on the device;
  * ``e2e``     - the same recipe through the public ``Trainer(TrainConfig).train()`` call: every micro-batch is
                  collated on the host, pinned, copied host->device inside the timed region, and the loss / gradient
                  norm are read back device->host every optimizer step.
``--impl reference`` runs the unmodified reference package (installed under ``baseline/_ref``) through its own
``Trainer`` on the same model, data shape and recipe.  One JSON line is printed by rank 0.
"""

from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

MODEL = dict(vocab_size=32000, hidden_size=2048, num_hidden_layers=24, rms_norm_eps=1e-6, intermediate_size=5632,
             tie_word_embeddings=True, max_position_embeddings=2048, rope_theta=10000.0, num_attention_heads=16,
             num_key_value_heads=4)
SEQ, BPD, ACCUM = 2048, 4, 8
LR, WD, SMOOTH, CLIP = 1e-4, 0.1, 0.05, 1.0
BASELINE_VALUE = None  # the reference publishes no training throughput

_DENSE_8B = dict(vocab_size=128256, hidden_size=4096, num_hidden_layers=32, rms_norm_eps=1e-5, intermediate_size=14336,
                 tie_word_embeddings=False, rope_theta=500000.0, num_attention_heads=32, num_key_value_heads=8)
_MOE_MLA = dict(vocab_size=32000, hidden_size=2048, num_hidden_layers=16, rms_norm_eps=1e-6, intermediate_size=1408,
                tie_word_embeddings=False, max_position_embeddings=4096, rope_theta=10000.0, num_attention_heads=16,
                num_key_value_heads=16, attn_type="mla", kv_lora_rank=512, q_lora_rank=1536, qk_nope_head_dim=128,
                qk_rope_head_dim=64, v_head_dim=128, ffn_type="moe", n_routed_experts=64, n_shared_experts=2,
                n_activated_experts=6, moe_intermediate_size=1408, shared_expert_intermediate_size=1408)

# The headline configuration (fsdp1b) and the three model-parallel configurations named beside it.  ``bpd`` is the batch a
# rank reads per micro-batch; ranks of one tp / cp block read the same batch, so the job's global batch is bpd x accum x
# data-parallel replicas.
CONFIGS = {
    "fsdp1b": dict(metric="train tok/s/box (1B dense FSDP)", label="1B dense decoder (24L d2048 16q/4kv hd128 ffn5632 v32000 tied)",
                   model=MODEL, seq=SEQ, bpd=BPD, accum=ACCUM, mode="fsdp", smooth=SMOOTH),
    "tp8b": dict(metric="train tok/s/box (8B dense TP, seq 8192, global batch 8)",
                 label="8B dense decoder (32L d4096 32q/8kv hd128 ffn14336 v128256 untied)",
                 model=dict(_DENSE_8B, max_position_embeddings=8192), seq=8192, bpd=8, accum=1, mode="tp", smooth=0.0),
    "cp8b": dict(metric="train tok/s/box (8B dense CP, seq 65536, batch 1)",
                 label="8B dense decoder (32L d4096 32q/8kv hd128 ffn14336 v128256 untied)",
                 model=dict(_DENSE_8B, max_position_embeddings=65536), seq=65536, bpd=1, accum=1, mode="cp", smooth=0.0),
    "ep_moe": dict(metric="train tok/s/box (MoE + MLA, EP, seq 4096, batch 2 per GPU)",
                   label="MoE decoder (16L d2048, MLA 16 heads kv_lora 512 q_lora 1536 nope 128 rope 64 v 128, "
                         "64 routed top-6 + 2 shared experts ffn 1408, v32000)",
                   model=_MOE_MLA, seq=4096, bpd=2, accum=1, mode="ep", smooth=0.0),
}


# ----------------------------------------------------------------------------------------------- clocks sampling
class ClockSampler:
    """Samples SM clocks and throttle reasons of this rank's GPU with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.path = index, None, None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "200", "-i", str(self.index)],
                stdout=fd, stderr=subprocess.DEVNULL)
            os.close(fd)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        clocks, reasons = [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        try:
            for line in open(self.path):
                parts = [p.strip() for p in line.split(",")]
                if len(parts) < 6 or not parts[0].isdigit():
                    continue
                clocks.append(int(parts[0]))
                out["sm_max_mhz"] = int(parts[1])
                for n, v in zip(names, parts[2:6]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
            os.unlink(self.path)
        except Exception:
            pass
        if clocks:
            out["sm_mhz"] = statistics.median(clocks)
        out["reasons"] = sorted(reasons)
        out["samples"] = len(clocks)
        return out


# ----------------------------------------------------------------------------------------------- shared pieces
def _dist_env():
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", rank))
    return rank, world, local


def _max_over_ranks(ms: float) -> float:
    import torch
    import torch.distributed as dist

    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        t = torch.tensor([ms], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())
    return ms


def _barrier_sync():
    import torch
    import torch.distributed as dist

    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        dist.barrier()
    torch.cuda.synchronize()


def _host_tokens(n, seq, vocab, seed=0):
    """Map-style dataset of packed uniform token ids living in host memory (seq strategy layout)."""
    import torch
    from torch.utils.data import Dataset

    class HostTokens(Dataset):
        def __init__(self):
            g = torch.Generator().manual_seed(seed)
            self.data = torch.randint(0, vocab, (n, seq + 1), generator=g)

        def __len__(self):
            return self.data.shape[0]

        def __getitem__(self, i):
            row = self.data[i]
            return {"input_ids": row[:-1], "target_ids": row[1:]}

    return HostTokens()


class _StepTimer:
    """Trainer callback: CUDA-event brackets around optimizer steps [W, W+K) counted in micro-batches."""

    def __init__(self, warmup, steps, accum, sampler=None):
        self.begin_at, self.end_at = warmup * accum, (warmup + steps) * accum
        self.seen = 0
        self.ms = None
        self.sampler = sampler
        self.launches = None
        self.count_fn = None
        self.host_syncs = []

    def on_batch_begin(self, context):
        import torch

        if self.seen == self.begin_at:
            _barrier_sync()
            if self.sampler:
                self.sampler.start()
            if self.count_fn:
                self._count0 = self.count_fn()
            self._e0 = torch.cuda.Event(enable_timing=True)
            self._e1 = torch.cuda.Event(enable_timing=True)
            self._e0.record()
        elif self.seen == self.end_at:
            self._e1.record()
            _barrier_sync()
            self.ms = _max_over_ranks(self._e0.elapsed_time(self._e1))
            if self.count_fn:
                self.launches = self.count_fn() - self._count0
            self.clocks = self.sampler.stop() if self.sampler else None
            context.request_stop()
        self.seen += 1

    def on_optimizer_step(self, context):
        # the step's results are read on the host every optimizer step (device->host inside the timed region)
        _ = context.loss
        _ = context.grad_norm


def _quiet_progress(callbacks):
    """Progress bars go to stderr so that stdout carries the JSON line only."""
    for cb in callbacks:
        if type(cb).__name__ == "ProgressBarCallback":
            cb.file = sys.stderr


def _spec(args):
    return CONFIGS[getattr(args, "config", "fsdp1b")]


def _replicas(spec, world):
    """Ranks that read different samples (the ranks of a tp / cp block share theirs)."""
    return 1 if spec["mode"] in ("tp", "cp") else world


def _emit(args, world, value_ms, e2e_ms, launches, clocks, impl, extra=None, note=None):
    spec = _spec(args)
    SEQ, BPD, ACCUM = spec["seq"], spec["bpd"], spec["accum"]
    readers = _replicas(spec, world)
    tokens_per_step = readers * BPD * ACCUM * SEQ
    value = tokens_per_step * args.steps / (value_ms / 1e3) if value_ms else None
    e2e = tokens_per_step * args.steps / (e2e_ms / 1e3) if e2e_ms else None
    line = {
        "metric": spec["metric"], "value": value if value is not None else e2e, "unit": "tokens/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": (value_ms or e2e_ms) / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None if not BASELINE_VALUE else (value or e2e) / BASELINE_VALUE,
        "dtype": f"fp8 ({args.fp8_recipe} scaling) linears, bf16 elsewhere" if getattr(args, "fp8_recipe", None) else "bf16",
        "data": "synthetic uniform token ids, random-init weights", "impl": impl,
        "config": {"model": spec["label"], "global_batch": readers * BPD * ACCUM,
                   "seq_len": SEQ, "batch_per_device": BPD, "grad_accum": ACCUM, "parallelism": f"{spec['mode']}{world}",
                   "optimizer": "AdamW lr1e-4 wd0.1", "label_smoothing": spec["smooth"], "max_grad_norm": CLIP,
                   "l2": "per-step working set (activations, weights, gradients > 10 GB) far exceeds the 126 MB L2; no explicit flush"},
        "clocks": clocks or {"sm_mhz": None, "sm_max_mhz": None, "reasons": []},
        "e2e": {"value": e2e, "unit": "tokens/s", "ms_per_step": (e2e_ms / args.steps) if e2e_ms else None,
                "h2d_bytes_per_step": ACCUM * BPD * SEQ * 8 * 2, "d2h_bytes_per_step": 8},
        "gpu_launches": launches,
    }
    line.update(extra or {})  # run facts that are not part of the benchmark's configuration (transport, last loss)
    if getattr(args, "smoke_layers", 0):
        line["invalid"] = f"smoke run with {args.smoke_layers} layers instead of the configuration's model"
    if note:
        line["note"] = note
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------------------------- our arm
def run_ours(args):
    import torch

    from astrai_b200.config import AutoRegressiveLMConfig, TrainConfig
    from astrai_b200.models import AutoRegressiveLM
    from astrai_b200.ops import native
    from astrai_b200.optim import FusedAdamW
    from astrai_b200.parallel.setup import setup_parallel
    from astrai_b200.trainer import SchedulerFactory, Trainer
    from astrai_b200.trainer.train_context import TrainContextBuilder

    rank, world, local = _dist_env()
    native.require()
    spec = _spec(args)
    seq, bpd, accum, mode = spec["seq"], spec["bpd"], spec["accum"], spec["mode"]
    if mode in ("tp", "cp", "ep") and world < 2:
        raise SystemExit(f"--config {args.config} is a model-parallel configuration: launch it on 2 or more GPUs")
    cfg = AutoRegressiveLMConfig(**dict(spec["model"], **({"num_hidden_layers": args.smoke_layers} if args.smoke_layers else {})))
    vocab = spec["model"]["vocab_size"]
    total_steps = args.warmup + args.steps
    big = cfg.hidden_size * cfg.num_hidden_layers >= 100_000  # 8B class: build on the GPU, the host would take minutes

    def model_fn():
        torch.manual_seed(1234)
        if big:
            with torch.device("cuda", local):
                return AutoRegressiveLM(cfg).to(torch.bfloat16)
        return AutoRegressiveLM(cfg).to(torch.bfloat16)

    if mode == "fsdp":
        exkw = {"comm": args.comm}
        if args.fsdp_reshard:  # full-shard placement (parameters / gradients whole only while their block computes)
            exkw = {"comm": "nccl", "reshard": True, "impl": "flat"}
    elif mode == "cp":
        exkw = {"comm": args.comm, "attn_comm": "nccl" if args.comm == "nccl" else "p2p", "max_tokens_per_rank": 2 * bpd * seq // world}
    elif mode == "ep":
        exkw = {"comm": "nccl" if args.comm == "nccl" else "p2p", "tokens_per_rank": bpd * seq}
    else:
        exkw = {"comm": "nccl" if args.comm == "nccl" else "p2p", "arena_bytes": 6 << 30}

    def make_config(dataset, ckpt_dir):
        return TrainConfig(
            model_fn=model_fn, strategy="seq", dataset=dataset,
            optimizer_fn=lambda m: FusedAdamW(m.parameters(), lr=LR, betas=(0.9, 0.999), weight_decay=WD),
            scheduler_fn=lambda o: SchedulerFactory.create("cosine", o, warmup_steps=2, lr_decay_steps=10_000),
            batch_per_device=bpd, grad_accum_steps=accum, max_grad_norm=CLIP, ckpt_dir=ckpt_dir, ckpt_interval=10**9,
            metrics=["loss", "lr", "grad_norm"], pin_memory=True, nprocs=world, parallel_mode=mode,
            strategy_kwargs={"label_smoothing": spec["smooth"]}, master_addr=os.environ.get("MASTER_ADDR", "127.0.0.1"),
            master_port=os.environ.get("MASTER_PORT", "29511"), executor_kwargs=exkw,
        )

    results = {}
    readers = _replicas(spec, world)
    reader = rank if readers == world else 0  # ranks of one tp / cp block read the same samples
    with setup_parallel(rank, world, local, "nccl", os.environ.get("MASTER_ADDR", "127.0.0.1"),
                        os.environ.get("MASTER_PORT", "29511"), "cuda"):
        dev = torch.device("cuda", local)
        # ---- (1) device-resident inputs: the step itself --------------------------------------------------------
        n_micro = total_steps * accum
        # one distinct micro-batch per timed / warm-up iteration: nothing repeats inside the run, so the loss stays
        # comparable with the end-to-end arm and with the reference arm (fresh uniform tokens every step)
        ds = _host_tokens(n_micro * bpd, seq, vocab, seed=1000 + reader)
        trainer = Trainer(make_config(ds, tempfile.mkdtemp(prefix="bench_ckpt_")), callbacks=[])
        trainer.callbacks = [cb for cb in trainer.callbacks if type(cb).__name__ in ("GradientClippingCallback",)]
        ctx = TrainContextBuilder(trainer.train_config).build()
        ctx.model.train()
        pool = [{k: ds.data[i * bpd:(i + 1) * bpd, sl].contiguous().to(dev)
                 for k, sl in (("input_ids", slice(0, seq)), ("target_ids", slice(1, seq + 1)))} for i in range(n_micro)]
        sampler = ClockSampler(local) if rank == 0 else None
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for i in range(n_micro):
            if i == args.warmup * accum:
                _barrier_sync()
                if sampler:
                    sampler.start()
                c0 = native.launch_count()
                e0.record()
            with ctx.executor.accumulate(ctx.model):
                trainer._micro_batch(ctx, pool[i])
        e1.record()
        _barrier_sync()
        results["value_ms"] = _max_over_ranks(e0.elapsed_time(e1))
        results["launches"] = native.launch_count() - c0
        results["clocks"] = sampler.stop() if sampler else None
        results["final_loss"] = ctx.loss
        results["peak_gb"] = round(torch.cuda.max_memory_allocated(dev) / 2**30, 1)
        assert native.kernel_status(dev) == 0, "a kernel's bounded wait expired"
        # a step that produced NaN / Inf runs at low power and high clocks: its timing is not a measurement
        if not math.isfinite(float(results["final_loss"])):
            raise RuntimeError(f"training diverged during the benchmark (loss {results['final_loss']}); no number is reported")
        if mode in ("tp", "cp", "ep"):  # the symmetric arenas of this context must go before a second one is built
            from astrai_b200.parallel import context_parallel, expert_parallel, tensor_parallel

            for mod in (tensor_parallel, context_parallel, expert_parallel):
                mod.set_context(None)
        del ctx, trainer, pool
        import gc

        gc.collect()
        torch.cuda.empty_cache()
        # ---- (2) end to end through Trainer.train(): host data, pinned H2D per micro-batch, D2H per step -----------
        if not args.skip_e2e:
            # the trainer's sampler deals the dataset out over the ranks: size it so that every rank has all its micro-batches
            host = _host_tokens((n_micro + 2) * bpd * readers, seq, vocab, seed=100)
            timer = _StepTimer(args.warmup, args.steps, accum)
            t2 = Trainer(make_config(host, tempfile.mkdtemp(prefix="bench_ckpt_")), callbacks=[timer])
            # keep the stock callbacks except the ones that write 2 GB checkpoints at exit
            t2.callbacks = [cb for cb in t2.callbacks if type(cb).__name__ not in ("CheckpointCallback", "MetricCallback")]
            _quiet_progress(t2.callbacks)
            t2.train()
            results["e2e_ms"] = timer.ms
    if rank == 0:
        _emit(args, world, results["value_ms"], results.get("e2e_ms"), results["launches"], results["clocks"], "ours",
              extra={"comm": "nccl" if args.fsdp_reshard else args.comm, "fsdp_placement": "full-shard" if args.fsdp_reshard else "replicated",
                     "final_loss": round(float(results["final_loss"]), 4), "peak_mem_gb": results["peak_gb"]})


# ----------------------------------------------------------------------------------------------- reference arm
def run_reference(args):
    if getattr(args, "config", "fsdp1b") != "fsdp1b":
        mode = _spec(args)["mode"]
        print(json.dumps({"impl": "reference", "unavailable": f"the reference has no {mode} parallel mode (its modes are none / ddp / fsdp); "
                          f"the comparison arm of --config {args.config} is this repository's own --comm nccl run"}))
        return
    ref_root = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_root, "astrai")):
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref/astrai is missing (offline install not present)"}))
        return
    sys.path.insert(0, ref_root)
    try:
        import torch
        from astrai.config import AutoRegressiveLMConfig, TrainConfig
        from astrai.model import AutoRegressiveLM
        from astrai.trainer import SchedulerFactory, Trainer
    except Exception as exc:  # noqa: BLE001
        print(json.dumps({"impl": "reference", "unavailable": f"reference import failed: {type(exc).__name__}: {exc}"[:300]}))
        return

    rank, world, local = _dist_env()
    cfg = AutoRegressiveLMConfig(**MODEL)
    total_steps = args.warmup + args.steps
    n_micro = total_steps * ACCUM
    sampler = ClockSampler(local) if rank == 0 else None
    timer = _StepTimer(args.warmup, args.steps, ACCUM, sampler)

    def model_fn():
        torch.manual_seed(1234)
        return AutoRegressiveLM(cfg).to(torch.bfloat16)  # the reference's train script casts the model to bf16

    def attempt(tied: bool):
        cfg.tie_word_embeddings = tied
        # the reference's sampler deals the dataset out over the ranks too: every rank needs all its micro-batches
        host = _host_tokens((n_micro + 2) * BPD * world, SEQ, MODEL["vocab_size"], seed=100)
        tc = TrainConfig(
            model_fn=model_fn, strategy="seq", dataset=host,
            optimizer_fn=lambda m: torch.optim.AdamW(m.parameters(), lr=LR, weight_decay=WD, fused=True),
            scheduler_fn=lambda o: SchedulerFactory.create("cosine", o, warmup_steps=2, lr_decay_steps=10_000),
            batch_per_device=BPD, grad_accum_steps=ACCUM, max_grad_norm=CLIP,
            ckpt_dir=tempfile.mkdtemp(prefix="ref_ckpt_"), ckpt_interval=10**9, metrics=["loss", "lr", "grad_norm"],
            pin_memory=True, nprocs=world, parallel_mode="fsdp", strategy_kwargs={"label_smoothing": SMOOTH},
            master_addr=os.environ.get("MASTER_ADDR", "127.0.0.1"), master_port=os.environ.get("MASTER_PORT", "29512"),
        )
        tr = Trainer(tc, callbacks=[timer])
        # stock callbacks stay, except the two that serialise a 2 GB checkpoint when training stops
        tr.callbacks = [cb for cb in tr.callbacks if type(cb).__name__ not in ("CheckpointCallback", "MetricCallback")]
        _quiet_progress(tr.callbacks)
        tr.train()

    note = None
    try:
        attempt(True)
    except Exception as exc:  # noqa: BLE001
        if world > 1 and timer.ms is None:
            note = f"tied embeddings failed under the reference's FSDP ({type(exc).__name__}); ran untied"
            timer.seen = 0
            attempt(False)
        else:
            raise
    if rank == 0:
        _emit(args, world, None, timer.ms, 0, getattr(timer, "clocks", None), "reference", note=note)


# ----------------------------------------------------------------------------------------------- serving mode
def run_serve_mode(args):
    """``--mode serve``: the continuous-batching load test of the 1B model (paged KV cache with 16-token pages, radix prefix
    cache, Poisson arrivals, log-normal prompts, 8 shared 1024-token prefixes, uniform output lengths, temperature 0.8 /
    top-p 0.95 / top-k 50, seed 0) through the scheduler's public API, for this framework or (``--impl reference``) for the
    unmodified reference package with the same request stream and the same ``max_batch_size``."""
    import torch

    from astrai_b200.cli import benchmark as B

    common = dict(n_requests=args.requests, rate=args.rate, max_batch_size=args.max_batch_size, max_seq_len=8192,
                  kv_cache_tokens=None, temperature=0.8, top_p=0.95, top_k=50, seed=0, time_scale=1.0)
    if args.impl == "reference":
        ref_root = os.path.join(ROOT, "baseline", "_ref")
        if not os.path.isdir(os.path.join(ref_root, "astrai")):
            print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref/astrai is missing (offline install not present)"}))
            return
        sys.path.insert(0, ref_root)
        import glob

        built = glob.glob(os.path.join(ref_root, "astrai", "extension", "lib", "*.so"))
        backend = args.ref_backend or ("cuda" if built else "flash")
        res = B._serve_reference("1b", "cuda", backend=backend, **common)
        launches = 0
    else:
        from astrai_b200.inference import InferenceScheduler
        from astrai_b200.ops import native

        native.require()
        model = B.build_model("1b", "cuda", torch.bfloat16)
        sched = InferenceScheduler(model, B._IdTokenizer(), max_batch_size=args.max_batch_size, max_seq_len=8192, page_size=16,
                                   kv_cache_tokens=args.max_batch_size * 4608, paged=True, chunked_prefill=True,
                                   max_prefill_tokens=8192)
        reqs = B.make_requests(args.requests, args.rate, model.config.vocab_size, 0)
        sched.run_batch([reqs[0]["ids"][:64]], max_tokens=4, temperature=0.0)  # warm-up (kernel load, graph capture)
        c0 = native.launch_count()
        sched.start()
        try:
            res = B.run_serve(sched, reqs, 0.8, 0.95, 50, 1.0)
        finally:
            sched.stop()
        launches = native.launch_count() - c0
        backend = "tcgen05"
    line = {
        "metric": "serve out tok/s (1B dense, paged KV 16 + radix, Poisson arrivals)", "value": res["output_tok_per_s"],
        "unit": "tokens/s", "n_gpus": 1, "steps": args.requests, "warmup": 1, "ms_per_step": None, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "impl": args.impl,
        "data": "synthetic request stream (seed 0), random-init weights",
        "ttft_ms_p50": res["ttft_ms_p50"], "ttft_ms_p99": res["ttft_ms_p99"], "tpot_ms_p50": res["tpot_ms_p50"],
        "completed": res["completed"], "wall_s": res["wall_s"], "output_tokens": res["output_tokens"],
        "prompt_tokens": res["prompt_tokens"], "gpu_launches": launches,
        "config": {"model": CONFIGS["fsdp1b"]["label"], "requests": args.requests, "rate_req_per_s": args.rate,
                   "max_batch_size": args.max_batch_size, "page_size": 16, "prefix_cache": "radix", "attention_backend": backend,
                   "prompt_len": "lognormal mean 512 sigma 0.6 in [16, 4096]; half share one of 8 prefixes of 1024",
                   "output_len": "uniform [64, 512]", "sampling": "temperature 0.8 top_p 0.95 top_k 50 seed 0"},
    }
    print(json.dumps(line), flush=True)


def _json_only_stdout():
    """Libraries print to stdout at times (NCCL's version banner); the contract is ONE JSON line there.  Everything
    written to file descriptor 1 from now on goes to stderr; ``print(json...)`` uses the saved descriptor."""
    import builtins

    real = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)
    sys.stdout = sys.stderr
    plain_print = builtins.print

    def emit(*a, **k):
        if a and isinstance(a[0], str) and a[0].startswith("{") and "file" not in k:
            k["file"] = real
            k["flush"] = True
        return plain_print(*a, **k)

    builtins.print = emit


def main():
    _json_only_stdout()
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=6)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--comm", default=os.environ.get("ASTRAI_B200_FSDP_COMM", "p2p"), choices=["nccl", "p2p", "nvls"],
                    help="transport: fused peer-memory kernels (p2p; nvls for FSDP) or NCCL collectives around the same math")
    ap.add_argument("--config", default="fsdp1b", choices=sorted(CONFIGS),
                    help="fsdp1b: the headline 1B FSDP run; tp8b / cp8b: 8B dense with tensor / context parallelism; "
                         "ep_moe: MoE + MLA with expert parallelism (these three need >= 2 GPUs)")
    ap.add_argument("--skip-e2e", action="store_true")
    ap.add_argument("--fp8-recipe", default=None, choices=["delayed", "dynamic", "block"],
                    help="run the linear layers on fp8 tensor cores with this scaling recipe (the line then says dtype fp8; "
                         "not the headline configuration, which is bf16)")
    ap.add_argument("--fsdp-reshard", action="store_true",
                    help="fsdp1b: the full-shard placement instead of the default replicated parameters + sharded optimizer state")
    ap.add_argument("--smoke-layers", type=int, default=0,
                    help="debugging aid: cut the model to this many layers (the line is then marked invalid, it is not a result)")
    ap.add_argument("--mode", default="train", choices=["train", "serve"],
                    help="serve: the continuous-batching load test (1 GPU) instead of a training step")
    ap.add_argument("--requests", type=int, default=2048)
    ap.add_argument("--rate", type=float, default=32.0, help="serve: Poisson arrival rate, requests per second")
    ap.add_argument("--max-batch-size", type=int, default=128)
    ap.add_argument("--ref-backend", default=None, help="serve, reference arm: its attention backend (default: cuda if built, else flash)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 1)
    if args.mode == "serve":
        try:
            run_serve_mode(args)
        except Exception as exc:  # noqa: BLE001
            if args.impl != "reference":
                raise
            why = f"the reference's own serving path failed on this box: {type(exc).__name__}: {exc}"
            print(json.dumps({"impl": "reference", "unavailable": " ".join(why.split())[:300]}), flush=True)
        return
    if args.impl == "reference":
        try:
            run_reference(args)
        except Exception as exc:  # noqa: BLE001 - the arm must end with a JSON line, not a traceback
            if int(os.environ.get("RANK", "0")) == 0:
                why = f"the reference's own code path failed on this box: {type(exc).__name__}: {exc}"
                print(json.dumps({"impl": "reference", "unavailable": " ".join(why.split())[:300]}), flush=True)
    elif args.fp8_recipe:
        from astrai_b200.ops import fp8

        recipe = {"delayed": fp8.DelayedScaling, "dynamic": fp8.DynamicScaling, "block": fp8.BlockScaling}[args.fp8_recipe]()
        with fp8.fp8_autocast(recipe=recipe):
            run_ours(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
