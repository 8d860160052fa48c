"""``python -m astrai_b200.cli.train``: build a :class:`TrainConfig` from options / YAML and run the trainer.

Option surface of the reference's ``scripts/tools/train.py:109-856`` (see its ``docs/guides/params.md``), plus the
knobs this framework adds: ``--parallel_mode tp|cp|ep`` with ``--tp_size / --cp_size / --ep_size`` select the model-parallel
executors (the reference parses ``--tp_size`` and drops it), ``--fsdp_comm`` / ``--mp_comm`` pick NCCL or the fused
peer-memory kernels,
``--fp8`` enables fp8 tensor-core linears, ``--optimizer fused_adamw`` selects the single-kernel AdamW.
"""

from __future__ import annotations

import json
import math
import os
from functools import partial
from typing import Any, Dict, Optional

import click

from astrai_b200.cli.common import flatten_sections, load_yaml, merge_config

SECTIONS = ("model", "data", "parallel", "training", "ckpt", "log", "optimizer", "scheduler", "rollout")


def compute_total_steps(n_samples: int, nprocs: int, batch_per_device: int, grad_accum_steps: int, n_epoch: int) -> int:
    """Optimizer steps of a run: ``ceil(ceil(N / nprocs) / bpd) // accum * epochs`` (reference ``train.py:603-617``)."""
    per_rank = math.ceil(n_samples / max(nprocs, 1))
    return max(math.ceil(per_rank / batch_per_device) // max(grad_accum_steps, 1), 1) * n_epoch


def optimizer_kwargs(o: Dict[str, Any]) -> Dict[str, Any]:
    name = o["optimizer"]
    kw: Dict[str, Any] = {"lr": o["max_lr"], "weight_decay": o["weight_decay"]}
    if name == "muon_adamw":
        kw.update(muon_momentum=o["muon_momentum"], muon_nesterov=o["muon_nesterov"], muon_ns_steps=o["muon_ns_steps"],
                  muon_adjust_lr=o["muon_adjust_lr"])
    elif name == "nora_nadamw":
        kw.update(nora_lr=o["nora_lr"], nora_beta=o["nora_beta"], nora_momentum=o["nora_momentum"],
                  nora_weight_decay=o["nora_weight_decay"])
    elif name == "mano_adamw":
        kw.update(mano_momentum=o["mano_momentum"], mano_nesterov=o["mano_nesterov"])
    return kw


def scheduler_kwargs(o: Dict[str, Any], total_steps: int) -> Dict[str, Any]:
    warmup = int(total_steps * o["warmup_ratio"])
    kw: Dict[str, Any] = {"warmup_steps": warmup}
    if o["min_rate"] is not None:
        kw["min_rate"] = o["min_rate"]
    rest = max(total_steps - warmup, 1)
    if o["schedule_type"] == "cosine":
        kw["lr_decay_steps"] = rest
    elif o["schedule_type"] == "sgdr":
        kw.update(cycle_length=o["cycle_length"] or rest, t_mult=o["t_mult"])
    elif o["schedule_type"] == "wsd":
        stable = o["stable_steps"] if o["stable_steps"] is not None else int(rest * 0.8)
        kw.update(stable_steps=stable, decay_steps=o["decay_steps"] if o["decay_steps"] is not None else max(rest - stable, 1))
    return kw


def strategy_kwargs(o: Dict[str, Any]) -> Dict[str, Any]:
    t = o["train_type"]
    if t in ("seq", "sft"):
        return {"label_smoothing": o["label_smoothing"]}
    if t in ("dpo", "online_dpo"):
        return {"beta": o["dpo_beta"]}
    return {"clip_eps": o["grpo_clip_eps"], "kl_coef": o["grpo_kl_coef"], "group_size": o["group_size"]}


def build_train_config(o: Dict[str, Any]):
    import torch

    from astrai_b200.config import AutoRegressiveLMConfig, TrainConfig
    from astrai_b200.data import DatasetFactory
    from astrai_b200.models import AutoRegressiveLM
    from astrai_b200.optim import OptimizerFactory
    from astrai_b200.trainer import SchedulerFactory

    model_cfg = AutoRegressiveLMConfig.from_file(os.path.join(o["param_path"], "config.json"))
    if o["neftune_alpha"]:
        model_cfg.neftune_alpha = o["neftune_alpha"]
    window = o["window_size"] or model_cfg.max_position_embeddings
    dataset = DatasetFactory.load(o["train_type"].replace("online_", ""), o["data_root_path"], window_size=window,
                                  stride=o["stride"], tokenizer_path=o["param_path"])
    from astrai_b200.parallel.mesh import data_parallel_size

    # ranks of one tensor- / context-parallel block read the same samples: they count once
    readers = data_parallel_size(o["parallel_mode"], o["nprocs"], o["tp_size"] or 1, o.get("cp_size") or 1, o.get("ep_size") or 1,
                                 o.get("pp_size") or 1)
    total_steps = compute_total_steps(len(dataset), readers, o["batch_per_device"], o["grad_accum_steps"], o["n_epoch"])
    opt_kw, sched_kw = optimizer_kwargs(o), scheduler_kwargs(o, total_steps)

    def model_fn():
        return AutoRegressiveLM(model_cfg).to(torch.bfloat16)

    executor_kwargs: Dict[str, Any] = {}
    if o["parallel_mode"] == "fsdp":
        executor_kwargs["comm"] = o["fsdp_comm"]
        if o.get("fsdp_reshard"):  # full-shard placement: library collectives, buffers released at rest
            executor_kwargs.update(comm="nccl", reshard=True, impl="flat")
    elif o["parallel_mode"] in ("tp", "ep"):
        executor_kwargs["comm"] = o.get("mp_comm") or "p2p"
    elif o["parallel_mode"] == "pp":
        if o.get("pp_chunks"):
            executor_kwargs["chunks"] = o["pp_chunks"]
    elif o["parallel_mode"] == "cp":
        executor_kwargs["attn_comm"] = o.get("mp_comm") or "p2p"
        executor_kwargs["comm"] = o["fsdp_comm"]
    from astrai_b200.models.decoder import DecoderBlock

    return TrainConfig(
        model_fn=model_fn, strategy=o["train_type"], dataset=dataset,
        optimizer_fn=partial(OptimizerFactory.create, o["optimizer"], **opt_kw), optimizer_name=o["optimizer"],
        optimizer_hyperparameters=opt_kw, scheduler_fn=lambda opt: SchedulerFactory.create(o["schedule_type"], opt, **sched_kw),
        n_epoch=o["n_epoch"], batch_per_device=o["batch_per_device"], grad_accum_steps=o["grad_accum_steps"],
        max_grad_norm=o["max_grad_norm"], gradient_checkpointing_modules=[DecoderBlock] if o["gradient_checkpointing"] else [],
        compile_mode=o["compile"], start_epoch=o["start_epoch"], start_samples=o["start_samples"], ckpt_dir=o["ckpt_dir"],
        ckpt_interval=o["ckpt_interval"], metrics=list(o["metrics"]), random_seed=o["random_seed"], num_workers=o["num_workers"],
        pin_memory=o["pin_memory"], persistent_workers=o.get("persistent_workers", True), moe_aux_loss_coef=o.get("moe_aux_loss_coef", 0.01),
        nprocs=o["nprocs"], backend=o["backend"], master_addr=o["master_addr"],
        master_port=str(o["master_port"]), parallel_mode=o["parallel_mode"], tp_size=o["tp_size"] or 1,
        cp_size=o.get("cp_size") or 1, ep_size=o.get("ep_size") or 1, pp_size=o.get("pp_size") or 1,
        start_method=o["start_method"], device_type=o["device_type"], val_split=o["val_split"], val_step=o["val_step"],
        neftune_alpha=o["neftune_alpha"], rollout_interval=o["rollout_interval"], rollout_temperature=o["rollout_temperature"],
        rollout_top_k=o["rollout_top_k"], rollout_top_p=o["rollout_top_p"], rollout_max_tokens=o["rollout_max_tokens"],
        executor_kwargs=executor_kwargs, strategy_kwargs=strategy_kwargs(o),
    ), total_steps


def plan(o: Dict[str, Any]) -> Dict[str, Any]:
    """What ``--dry-run`` prints: the merged options that matter, without touching data or devices."""
    keys = ("train_type", "data_root_path", "param_path", "resume", "n_epoch", "batch_per_device", "grad_accum_steps",
            "max_lr", "warmup_ratio", "max_grad_norm", "optimizer", "weight_decay", "schedule_type", "window_size", "stride",
            "ckpt_dir", "ckpt_interval", "nprocs", "parallel_mode", "fsdp_comm", "fsdp_reshard", "tp_size", "cp_size", "ep_size",
            "pp_size", "pp_chunks", "mp_comm", "backend", "fp8", "fp8_recipe", "metrics",
            "label_smoothing", "gradient_checkpointing", "random_seed")
    out = {k: (list(o[k]) if isinstance(o[k], tuple) else o[k]) for k in keys}
    out["tokens_per_optimizer_step"] = o["batch_per_device"] * o["grad_accum_steps"] * o["nprocs"] * (o["window_size"] or 0)
    return out


@click.command(context_settings={"show_default": True, "max_content_width": 110})
@click.option("--config", "-c", type=click.Path(exists=True, dir_okay=False), default=None,
              help="YAML file; explicit options win.")
# basic
@click.option("--train_type", type=click.Choice(["seq", "sft", "dpo", "grpo", "online_grpo", "online_dpo"]), default=None,
              help="Objective: next-token (seq), masked supervised (sft), preference pairs (dpo), groups of scored responses "
                   "(grpo), or the last two with responses sampled during training (online_*).")
@click.option("--data_root_path", type=str, default=None,
              help="Directory written by the preprocessing step (or raw .jsonl files for sft / dpo).")
@click.option("--param_path", type=str, default=None, help="Model directory (config.json [+ weights]) or checkpoint.")
@click.option("--resume/--no-resume", default=False,
              help="Continue the run whose checkpoint --param_path names: optimizer, scheduler, epoch and position in the "
                   "data.")
@click.option("--n_epoch", type=int, default=1, help="Passes over the data.")
@click.option("--batch_per_device", type=int, default=1, help="Samples per micro-batch on every data-parallel rank.")
@click.option("--grad_accum_steps", type=int, default=1, help="Micro-batches per optimizer step.")
# learning rate / clipping
@click.option("--warmup_ratio", type=float, default=0.05, help="Share of all optimizer steps spent on linear warm-up.")
@click.option("--max_lr", type=float, default=3e-4, help="Peak learning rate.")
@click.option("--max_grad_norm", type=click.FloatRange(min=0, min_open=True), default=1.0, help="Gradient-norm clip.")
# optimizer
@click.option("--optimizer", type=click.Choice(["muon_adamw", "nora_nadamw", "mano_adamw", "fused_adamw"]), default="muon_adamw",
              help="muon_adamw / nora_nadamw / mano_adamw: a matrix rule on the decoder blocks' 2-D weights, AdamW or NAdamW "
                   "elsewhere; fused_adamw: AdamW everywhere, one kernel per parameter buffer.")
@click.option("--weight_decay", type=float, default=0.1,
              help="Decoupled weight decay (not applied to norms, biases and embeddings by the composite optimizers).")
@click.option("--muon_momentum", type=float, default=0.95, help="muon_adamw: momentum.")
@click.option("--muon_nesterov/--no-muon_nesterov", default=True, help="muon_adamw: Nesterov momentum.")
@click.option("--muon_ns_steps", type=int, default=5, help="muon_adamw: Newton-Schulz iterations of the orthogonalisation.")
@click.option("--muon_adjust_lr", type=click.Choice(["original", "match_rms_adamw"]), default="match_rms_adamw",
              help="muon_adamw: learning-rate scaling per matrix shape.")
@click.option("--nora_lr", type=float, default=5e-3, help="nora_nadamw: learning rate of the matrix rule.")
@click.option("--nora_beta", type=float, default=0.95, help="nora_nadamw: second-moment decay of the matrix rule.")
@click.option("--nora_momentum", type=float, default=0.95, help="nora_nadamw: momentum of the matrix rule.")
@click.option("--nora_weight_decay", type=float, default=0.0, help="nora_nadamw: weight decay of the matrix rule.")
@click.option("--mano_momentum", type=float, default=0.95, help="mano_adamw: momentum.")
@click.option("--mano_nesterov/--no-mano_nesterov", default=True, help="mano_adamw: Nesterov momentum.")
# scheduler
@click.option("--schedule_type", type=click.Choice(["cosine", "sgdr", "wsd"]), default="cosine",
              help="Learning-rate curve after the warm-up.")
@click.option("--min_rate", type=float, default=None,
              help="Floor of the curve as a fraction of --max_lr (default: the scheduler's own).")
@click.option("--cycle_length", type=int, default=None,
              help="sgdr: steps of the first cycle (default: all steps after the warm-up).")
@click.option("--t_mult", type=int, default=2, help="sgdr: every cycle is this many times longer than the one before.")
@click.option("--stable_steps", type=int, default=None,
              help="wsd: steps at --max_lr (default: 80 % of the steps after the warm-up).")
@click.option("--decay_steps", type=int, default=None, help="wsd: steps of the final decay (default: the rest).")
# data
@click.option("--window_size", type=int, default=None,
              help="Tokens per training sample (default: the model's max_position_embeddings).")
@click.option("--stride", type=int, default=None,
              help="seq / sft: distance between the starts of two windows (default: the window).")
@click.option("--random_seed", type=int, default=3407, help="Seed of the shuffling and of the validation split.")
@click.option("--num_workers", type=int, default=4, help="Data-loader worker processes.")
@click.option("--pin_memory/--no-pin_memory", default=True, help="Page-locked host batches.")
@click.option("--persistent_workers/--no-persistent_workers", default=True,
              help="Keep the data-loader workers alive between epochs.")
# checkpoints / validation / logging
@click.option("--ckpt_interval", type=int, default=5000, help="Optimizer steps between checkpoints.")
@click.option("--ckpt_dir", type=str, default="checkpoint", help="Where checkpoints and metric logs go.")
@click.option("--start_epoch", type=int, default=0, help="Epoch to start counting from (without --resume).")
@click.option("--start_samples", type=int, default=0, help="Samples per rank to skip in the first epoch (without --resume).")
@click.option("--val_split", type=float, default=None, help="Hold this fraction of the data out and log its loss.")
@click.option("--val_step", type=int, default=1000, help="Optimizer steps between validation passes.")
@click.option("--metrics", multiple=True, default=("loss", "lr", "grad_norm", "grad_snr"),
              help="Columns of metric.jsonl: loss, lr, grad_norm, grad_snr, val_loss, moe_aux_loss, router_entropy, "
                   "dead_expert_fraction, load_imbalance_mean, load_imbalance_max.")
@click.option("--gradient_checkpointing/--no-gradient_checkpointing", default=False,
              help="Recompute every decoder block in the backward pass.")
@click.option("--compile", type=click.Choice(["default", "reduce-overhead", "max-autotune"]), default=None,
              help="Wrap the model in torch.compile with this mode (kept for configs of the reference; off by default, the "
                   "kernels here are hand-written).")
@click.option("--dry-run", "dry_run", is_flag=True, default=False, help="Validate and print the plan; do not train.")
# distributed
@click.option("--nprocs", type=int, default=1, help="Ranks to spawn on this node (ignored under torchrun).")
@click.option("--parallel_mode", type=click.Choice(["none", "ddp", "fsdp", "tp", "cp", "ep", "pp"]), default="fsdp",
              help="tp / cp / ep / pp: tensor-, context-, expert- or pipeline-parallel blocks of --tp_size / --cp_size / "
                   "--ep_size / --pp_size ranks.")
@click.option("--fsdp_comm", type=click.Choice(["nccl", "p2p", "nvls"]), default="p2p",
              help="FSDP transport: NCCL or fused peer-memory kernels.")
@click.option("--fsdp_reshard", is_flag=True, default=False,
              help="FSDP full-shard placement: parameters and gradients are whole only while their block computes "
                   "(gathers and reduce-scatters every micro-batch; NCCL transport).")
@click.option("--device_type", type=str, default="cuda", help="cuda, or cpu for debugging with --backend gloo.")
@click.option("--start_method", type=click.Choice(["spawn", "fork", "forkserver"]), default="spawn",
              help="How local ranks are started.")
@click.option("--backend", type=click.Choice(["nccl", "gloo"]), default="nccl", help="torch.distributed backend.")
@click.option("--master_addr", type=str, default="127.0.0.1", help="Rendezvous address.")
@click.option("--master_port", type=int, default=29500, help="Rendezvous port.")
@click.option("--tp_size", type=int, default=None,
              help="Tensor-parallel size inside one NVSwitch domain (<= 8); default: all ranks.")
@click.option("--cp_size", type=int, default=None,
              help="Context-parallel size (ranks that share one sequence); default: all ranks.")
@click.option("--ep_size", type=int, default=None,
              help="Expert-parallel size (ranks that share one set of experts); default: all ranks.")
@click.option("--pp_size", type=int, default=None,
              help="Pipeline stages (ranks that hold one model replica layer range by layer range); default: all ranks. "
                   "Trains --train_type seq, sft, dpo and grpo.")
@click.option("--pp_chunks", type=int, default=None,
              help="pp: pieces a per-device batch is cut into for the 1F1B schedule (default: the number of stages, at most "
                   "the batch).")
@click.option("--mp_comm", type=click.Choice(["p2p", "nccl"]), default="p2p",
              help="tp / cp / ep transport: fused peer-memory kernels or library collectives around the same math.")
@click.option("--fp8/--no-fp8", default=False, help="Run linear layers on fp8 tensor cores.")
@click.option("--fp8_recipe", type=click.Choice(["delayed", "dynamic", "block"]), default="delayed",
              help="fp8 scaling: per-tensor from the amax history, per-tensor measured on the tensor, or per 1x128 / 128x128 block.")
# strategy specific
@click.option("--dpo_beta", type=float, default=0.1, help="dpo: strength of the preference margin.")
@click.option("--label_smoothing", type=float, default=0.0, help="seq / sft: label smoothing of the cross-entropy.")
@click.option("--group_size", type=int, default=4, help="grpo: responses per prompt.")
@click.option("--grpo_clip_eps", type=float, default=0.2, help="grpo: clip range of the probability ratio.")
@click.option("--grpo_kl_coef", type=float, default=0.01, help="grpo: weight of the KL term against the reference model.")
@click.option("--moe_aux_loss_coef", type=float, default=0.01,
              help="Weight of the mixture-of-experts load-balancing loss (0 = off).")
@click.option("--neftune_alpha", type=float, default=0.0, help="NEFTune noise on the embeddings while training (0 = off).")
# rollout
@click.option("--rollout_interval", type=int, default=512, help="online_*: samples between two rounds of generation.")
@click.option("--rollout_temperature", type=float, default=0.7, help="online_*: sampling temperature.")
@click.option("--rollout_top_k", type=int, default=0, help="online_*: top-k (0 = off).")
@click.option("--rollout_top_p", type=float, default=0.9, help="online_*: top-p.")
@click.option("--rollout_max_tokens", type=int, default=1024, help="online_*: longest sampled response.")
@click.pass_context
def train_command(ctx: click.Context, config: Optional[str], **opts):
    """Train a decoder LM (seq / sft / dpo / grpo, offline or with online rollouts)."""
    merged = merge_config(ctx, opts, flatten_sections(load_yaml(config), SECTIONS))
    missing = [k for k in ("train_type", "data_root_path", "param_path") if not merged.get(k)]
    if missing:
        raise click.UsageError("missing required option(s): " + ", ".join("--" + m for m in missing))
    if merged["dry_run"]:
        click.echo(json.dumps(plan(merged), indent=2, default=str))
        return
    train(**merged)


def train(**o):
    from astrai_b200.ops import fp8 as fp8_mod
    from astrai_b200.trainer import Trainer

    cfg, total_steps = build_train_config(o)
    click.echo(f"training plan: {total_steps} optimizer steps, parallel_mode={cfg.parallel_mode}, nprocs={cfg.nprocs}")
    trainer = Trainer(cfg)
    if o.get("fp8"):
        recipes = {"delayed": fp8_mod.DelayedScaling, "dynamic": fp8_mod.DynamicScaling, "block": fp8_mod.BlockScaling}
        recipe = recipes[o.get("fp8_recipe") or "delayed"]()
        with fp8_mod.fp8_autocast(recipe=recipe):
            trainer.train(o["param_path"], resume=o["resume"])
    else:
        trainer.train(o["param_path"], resume=o["resume"])


if __name__ == "__main__":
    train_command()
