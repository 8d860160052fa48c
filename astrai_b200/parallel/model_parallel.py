"""Training executors for the model-parallel modes: ``tp`` (tensor + sequence parallel), ``cp`` (context parallel,
zig-zag sequence sharding) and ``ep`` (expert parallel).

The reference accepts ``--tp_size`` and silently drops it (``scripts/tools/train.py:513-519``, ``:549-550``) and knows
the modes ``none | ddp | fsdp`` only (``astrai/config/train_config.py:15``).  Here ``parallel_mode = "tp" | "cp" | "ep"``
with ``tp_size / cp_size / ep_size`` selects one of the executors below through the same ``ExecutorFactory`` the
trainer already uses.  All three run on the flat-buffer runtime (fp32 ``main_grad`` filled by the wgrad kernels, clip
coefficient on the device, fused AdamW) and differ in

* how the model is rewritten at wrap time (``tp``: attention / FFN blocks become their sharded forms; ``ep``: the routed
  experts of every MoE layer become this rank's stacked share; ``cp``: nothing, the attention op is swapped by a context),
* how a batch is cut for this rank (:meth:`shard_batch`, called by the strategies),
* over which ranks a parameter's gradient is summed (replicated parameters: every rank; sharded ones: the ranks that
  hold the same shard) - units of the flat engine are split by that property,
* how the full state dict is put back together for checkpoints (reference keys and shapes).

Ranks are laid out by :mod:`astrai_b200.parallel.mesh`: blocks of ``mp_size`` consecutive ranks form one model-parallel
group; ``world / mp_size`` such blocks are data-parallel replicas (``tp``, ``cp``) or further expert-parallel groups
working on their own data (``ep``).  Every rank's loss is the mean over its own tokens, so a uniform ``1 / world`` factor
(folded into the clip coefficient) turns the summed gradients into the gradient of the global mean loss.
``comm="p2p"`` uses the fused peer-memory kernels, ``comm="nccl"`` library collectives around the same math (the
baseline arm, and the CPU / Gloo path of the tests).
"""

from __future__ import annotations

import logging
from typing import Dict, Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from astrai_b200.parallel.executor import ExecutorFactory, FlatExecutor, FSDPExecutor
from astrai_b200.parallel.flat import FlatParamEngine, FlatUnit
from astrai_b200.parallel.mesh import ParallelMesh, build_mesh
from astrai_b200.parallel.setup import get_rank, get_world_size

logger = logging.getLogger(__name__)

REPLICATED, SHARDED = "rep", "shard"


class ModelParallelExecutor(FlatExecutor):
    """Shared machinery of ``tp`` and ``ep``: flat runtime, two gradient-reduction groups, group-aware gradient norm."""

    communicates_every_micro_batch = True
    mode = ""

    def __init__(self, grad_accum_steps: int = 1, size: int = 0, comm: str = "p2p", overlap: bool = True,
                 comm_timeout_s: float = 120.0, arena_bytes: Optional[int] = None):
        super().__init__(grad_accum_steps, impl="flat", overlap=overlap)
        if comm not in ("p2p", "nccl"):
            raise ValueError("comm must be 'p2p' or 'nccl'")
        self.size, self.comm, self.comm_timeout_s, self.arena_bytes = int(size), comm, float(comm_timeout_s), arena_bytes
        self.mesh: Optional[ParallelMesh] = None

    # -- to be provided by the modes -------------------------------------------------------------------------------------
    def _convert(self, model: nn.Module) -> nn.Module:
        raise NotImplementedError

    def _is_sharded(self, name: str, p: nn.Parameter) -> bool:
        raise NotImplementedError

    def _full_state_dict(self, model: nn.Module) -> Optional[Dict[str, torch.Tensor]]:
        raise NotImplementedError

    def shard_batch(self, batch: dict) -> dict:
        return batch

    @property
    def data_parallel_size(self) -> int:
        return get_world_size()

    @property
    def data_parallel_rank(self) -> int:
        return get_rank()

    # -- set-up -------------------------------------------------------------------------------------------------------------
    def _prepare_model(self, model: nn.Module) -> nn.Module:
        self.mesh = build_mesh(self.size if self.size > 1 else None)
        on_gpu = next(model.parameters()).is_cuda
        if not on_gpu and self.comm == "p2p":
            self.comm = "nccl"  # the fused kernels need CUDA peer memory; on CPU the collective arm is the only one
        if self.use_distributed:  # one set of initial weights everywhere before anything is cut
            for t in list(model.parameters()) + list(model.buffers()):
                dist.broadcast(t.data, src=0)
        model = self._convert(model)
        self.engine = FlatParamEngine(model, 1, 0, tag_fn=lambda n, p: SHARDED if self._is_sharded(n, p) else REPLICATED)
        model._flat_engine, model._flat_executor = self.engine, self
        if self.use_distributed and on_gpu:
            self._comm_stream = torch.cuda.Stream()
        for unit in self.engine.units:
            for mname in unit.module_names:
                model.get_submodule(mname).register_forward_pre_hook(self._make_pre_hook(unit), with_kwargs=True)
        return model

    # -- gradients ---------------------------------------------------------------------------------------------------------
    def _group_for(self, unit: FlatUnit):
        """(process group, whether a reduction is needed) for this unit's gradient."""
        m = self.mesh
        if unit.tag == REPLICATED:
            return None, m.world > 1                                    # every rank (WORLD)
        return m.dp_group, (m.dp_size > 1 and m.mp_size < m.world)      # ranks holding the same shard

    def _reduce_unit(self, unit: FlatUnit):
        unit.reduced = True
        group, needed = self._group_for(unit)
        if not needed or not self.use_distributed:
            return
        if self._comm_stream is not None:
            self._comm_stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self._comm_stream):
                dist.all_reduce(unit.grad_buf, group=group)
        else:
            dist.all_reduce(unit.grad_buf, group=group)

    def _averaging_scale(self) -> float:
        return 1.0 / get_world_size() if self.use_distributed else 1.0

    def _grad_sumsq(self) -> torch.Tensor:
        """Squared norm of the whole (unsharded) gradient: replicated units count once, sharded units are summed over
        the model-parallel group."""
        from astrai_b200 import ops

        dev = self.engine.units[0].grad_buf.device
        rep = torch.zeros(1, dtype=torch.float32, device=dev)
        shard = torch.zeros(1, dtype=torch.float32, device=dev)
        for u in self.engine.units:
            ops.sumsq(u.grad_buf, rep if u.tag == REPLICATED else shard)
        if self.use_distributed and self.mesh.mp_size > 1:
            dist.all_reduce(shard, group=self.mesh.mp_group)
        return rep + shard

    # -- state ------------------------------------------------------------------------------------------------------------
    def unwrap_model(self, model: nn.Module):
        return self._full_state_dict(model)

    def local_state_dict(self, model: nn.Module):
        return None  # parts of the model live on other ranks


@ExecutorFactory.register("tp")
class TensorParallelExecutor(ModelParallelExecutor):
    """``parallel_mode="tp"``: Megatron-style tensor parallelism with sequence-sharded activations inside blocks of
    ``tp_size`` ranks (:mod:`astrai_b200.parallel.tp_model`), data parallelism across the blocks.

    Every rank of a block reads the same batch; rank ``r`` keeps token rows ``[r*T/tp, (r+1)*T/tp)`` between the layers
    and computes the loss on those rows, so per-token tensors of the batch other than ``input_ids`` / ``position_ids``
    are cut to those rows by :meth:`shard_batch`.  Objectives over whole sequences (DPO, GRPO) keep the batch whole on
    every rank: each rank scores its token rows and the per-token log-probabilities are gathered over the block
    (``trainer/strategy.py::token_logprobs``), so every rank evaluates the same loss; the frozen reference / behaviour
    models are whole replicas."""

    mode = "tp"
    PER_TOKEN = ("target_ids", "loss_mask")

    def _convert(self, model):
        from astrai_b200.parallel import tensor_parallel as tpar
        from astrai_b200.parallel.tp_model import shard_model_

        m = self.mesh
        if m.mp_size > 1:
            tpar.set_group(m.mp_group, m.mp_rank, m.mp_size)
            if self.comm == "p2p":
                ctx = tpar.init_tensor_parallel(self.arena_bytes or (2 << 30), timeout_s=self.comm_timeout_s, group=m.mp_group)
                ctx.group = m.mp_group
        else:
            tpar.set_group(None, 0, 1)
        return shard_model_(model, m.mp_size, m.mp_rank, comm=self.comm)

    def _is_sharded(self, name, p):
        from astrai_b200.parallel.tp_model import is_sharded

        return is_sharded(name)

    @property
    def data_parallel_size(self):
        return self.mesh.dp_size if self.mesh else 1

    @property
    def data_parallel_rank(self):
        return self.mesh.dp_rank if self.mesh else 0

    @staticmethod
    def _widen(t: torch.Tensor, width: int) -> torch.Tensor:
        return t if t.shape[-1] == width else torch.nn.functional.pad(t, (0, width - t.shape[-1]))

    def pad_sequences(self, batch):
        """Sequence-level batches (preference pairs, response groups) keep whole sequences on every rank, but the model
        still cuts the batch's ``rows x length`` tokens into equal row blocks: widen the sequences with padding (id 0,
        mask 0) until the token count divides over the block.  Called by the strategies before they build masks."""
        tp = self.mesh.mp_size if self.mesh is not None else 1
        if tp <= 1:
            return batch
        out = dict(batch)
        if "chosen" in batch and "rejected" in batch:
            rows, length = 2 * batch["chosen"].shape[0], max(batch["chosen"].shape[1], batch["rejected"].shape[1])
            while rows * length % tp:
                length += 1
            for key in ("chosen", "rejected", "chosen_mask", "rejected_mask"):
                out[key] = self._widen(batch[key], length)
        elif "responses" in batch and "prompts" in batch:
            b, g, rlen = batch["responses"].shape
            plen = batch["prompts"].shape[1]
            while b * g * (plen + rlen) % tp:
                rlen += 1
            for key in ("responses", "masks"):
                out[key] = self._widen(batch[key], rlen)
        return out

    def shard_batch(self, batch):
        if "input_ids" not in batch or "target_ids" not in batch:
            if ("chosen" in batch and "rejected" in batch) or ("responses" in batch and "prompts" in batch):
                return batch  # whole sequences everywhere: the model cuts token rows itself, log-probabilities are gathered
            raise NotImplementedError("tensor parallelism takes token-level batches (input_ids / target_ids), preference pairs "
                                      f"(chosen / rejected) or response groups (prompts / responses); got keys {sorted(batch)}")
        tp, r = self.mesh.mp_size, self.mesh.mp_rank
        out = dict(batch)
        for key in self.PER_TOKEN:
            t = batch.get(key)
            if isinstance(t, torch.Tensor):
                flat = t.reshape(-1)
                local = flat.numel() // tp
                out[key] = flat[r * local:(r + 1) * local]
        if isinstance(batch.get("loss_mask"), torch.Tensor) and tp > 1:
            # a masked mean: every rank divides by 1/tp of the batch's trained tokens, so that the average over the block
            # is the mean over all of them (the ranks' own counts differ)
            out["loss_denominator"] = batch["loss_mask"].bool().sum().float() / tp
        return out

    def _full_state_dict(self, model):
        from astrai_b200.parallel.tp_model import gather_state_dict

        sd = gather_state_dict(model, group=self.mesh.mp_group)
        return sd if get_rank() == 0 else None


@ExecutorFactory.register("ep")
class ExpertParallelExecutor(ModelParallelExecutor):
    """``parallel_mode="ep"``: the routed experts of every MoE layer are spread over blocks of ``ep_size`` ranks
    (:class:`~astrai_b200.parallel.expert_parallel.EPExperts`); everything else is replicated and every rank trains on
    its own batch, so non-expert gradients are summed over all ranks and expert gradients over the ranks that hold the
    same experts."""

    mode = "ep"

    def __init__(self, grad_accum_steps: int = 1, size: int = 0, comm: str = "p2p", overlap: bool = True,
                 comm_timeout_s: float = 120.0, arena_bytes: Optional[int] = None, capacity_factor: Optional[float] = 2.0,
                 tokens_per_rank: Optional[int] = None):
        super().__init__(grad_accum_steps, size, comm, overlap, comm_timeout_s, arena_bytes)
        self.capacity_factor, self.tokens_per_rank = capacity_factor, tokens_per_rank

    def _convert(self, model):
        from astrai_b200.models.ffn import DeepSeekMoE
        from astrai_b200.parallel import expert_parallel as epar

        m = self.mesh
        layers = [mod for mod in model.modules() if isinstance(mod, DeepSeekMoE)]
        if not layers:
            raise ValueError("parallel_mode='ep' needs a model with MoE layers (ffn_type='moe')")
        if m.mp_size > 1 and self.comm == "p2p":
            first = layers[0]
            hidden = first.dim
            tokens = self.tokens_per_rank or 8192
            need = self.arena_bytes or epar.arena_bytes_for(tokens, hidden, first.n_activated_experts, m.mp_size,
                                                            first.n_routed_experts, self.capacity_factor)
            epar.init_expert_parallel(need, timeout_s=self.comm_timeout_s, group=m.mp_group)
        for moe in layers:
            experts = epar.EPExperts(moe.routed_experts, m.mp_size, m.mp_rank, comm=self.comm if m.mp_size > 1 else "nccl",
                                     group=m.mp_group, capacity_factor=self.capacity_factor)
            moe.routed_experts = experts
            moe.expert_parallel = True
        return model

    def _is_sharded(self, name, p):
        return ".routed_experts." in name

    def _full_state_dict(self, model):
        m = self.mesh
        first = get_rank() == 0
        out = {}
        for name, t in model.state_dict().items():
            if ".routed_experts." not in name:
                if first:
                    out[name] = t
                continue
            parts = [torch.empty_like(t) for _ in range(m.mp_size)]
            if m.mp_size > 1:
                dist.all_gather(parts, t.contiguous(), group=m.mp_group)
            else:
                parts = [t]
            if first:
                out[name] = torch.cat(parts, dim=0)
        if not first:
            return None
        # stacked [E, ...] tensors back to the reference's per-expert keys
        final = {k: v for k, v in out.items() if ".routed_experts." not in k}
        prefixes = sorted({k.rsplit(".", 1)[0] for k in out if k.endswith(".routed_experts.gate_up")})
        for pre in prefixes:
            gate_up, down = out[pre + ".gate_up"], out[pre + ".down"]
            f = gate_up.shape[1] // 2
            for j in range(gate_up.shape[0]):
                final[f"{pre}.{j}.gate.weight"] = gate_up[j, :f].contiguous()
                final[f"{pre}.{j}.up.weight"] = gate_up[j, f:].contiguous()
                final[f"{pre}.{j}.down.weight"] = down[j].contiguous()
        return final


@ExecutorFactory.register("cp")
class ContextParallelExecutor(FSDPExecutor):
    """``parallel_mode="cp"``: every sequence is cut zig-zag over blocks of ``cp_size`` ranks; attention fetches the other
    ranks' keys inside its kernel (:mod:`astrai_b200.parallel.context_parallel`).

    Parameters are replicated over all ranks, so everything outside attention is the flat FSDP runtime unchanged
    (gradients reduce-scattered over all ranks, optimizer state sharded, parameters gathered after the update): a long
    sequence costs activation memory, and sharding the optimizer state is what leaves room for it.  Only the token-level
    objectives (seq, and sft without packed-document masks) can be sequence-sharded."""

    communicates_every_micro_batch = True
    mode = "cp"
    PER_TOKEN = ("input_ids", "target_ids", "loss_mask")

    def __init__(self, grad_accum_steps: int = 1, size: int = 0, comm: str = "p2p", attn_comm: Optional[str] = None,
                 overlap: bool = True, comm_timeout_s: float = 120.0, arena_bytes: Optional[int] = None,
                 max_tokens_per_rank: Optional[int] = None, impl: str = "flat"):
        super().__init__(grad_accum_steps, impl=impl, overlap=overlap, comm=comm, comm_timeout_s=comm_timeout_s)
        self.size, self.attn_comm, self.arena_bytes = int(size), attn_comm or ("nccl" if comm == "nccl" else "p2p"), arena_bytes
        self.max_tokens_per_rank = max_tokens_per_rank
        self.mesh: Optional[ParallelMesh] = None
        self._cp = None

    def _prepare_model(self, model):
        from astrai_b200.parallel import context_parallel as cpar

        self.mesh = build_mesh(self.size if self.size > 1 else None)
        m = self.mesh
        on_gpu = next(model.parameters()).is_cuda
        if m.mp_size > 1 and on_gpu:
            cfg = model.config
            head_dim = cfg.hidden_size // cfg.num_attention_heads
            tokens = self.max_tokens_per_rank or cfg.max_position_embeddings // m.mp_size * 4
            need = self.arena_bytes or cpar.arena_bytes_for(1, tokens * m.mp_size, m.mp_size, cfg.num_key_value_heads, head_dim)
            self._cp = cpar.init_context_parallel(need, timeout_s=self.comm_timeout_s, group=m.mp_group)
            self._cp.comm = self.attn_comm
        elif m.mp_size > 1:
            self._cp = cpar.init_context_parallel_group(m.mp_group)
        return super()._prepare_model(model)

    @property
    def data_parallel_size(self):
        return self.mesh.dp_size if self.mesh else 1

    @property
    def data_parallel_rank(self):
        return self.mesh.dp_rank if self.mesh else 0

    def shard_batch(self, batch):
        from astrai_b200.parallel.context_parallel import zigzag_positions, zigzag_split

        if "input_ids" not in batch or "target_ids" not in batch:
            raise NotImplementedError("context parallelism shards token-level objectives (seq); this batch has no "
                                      "input_ids / target_ids pair")
        if "position_ids" in batch:
            raise NotImplementedError("packed documents (position_ids in the batch) are not sequence-sharded: attention "
                                      "across the ranks is plain causal")
        cp, r = self.mesh.mp_size, self.mesh.mp_rank
        if cp == 1:
            return batch
        out = dict(batch)
        b, s = batch["input_ids"].shape
        for key in self.PER_TOKEN:
            t = batch.get(key)
            if isinstance(t, torch.Tensor):
                out[key] = zigzag_split(t, cp, r, dim=1).contiguous()
        out["position_ids"] = zigzag_positions(s, cp, r, device=batch["input_ids"].device).unsqueeze(0).expand(b, -1)
        return out


@ExecutorFactory.register("pp")
class PipelineParallelExecutor(ModelParallelExecutor):
    """``parallel_mode="pp"``: the decoder is cut into ``pp_size`` contiguous layer ranges (:mod:`astrai_b200.parallel.pipeline`);
    rank ``r`` of a block holds stage ``r`` only, the blocks are data-parallel replicas.

    Every rank of a block reads the same batch (the first stage uses the token ids, the last one the targets).  One
    trainer micro-batch is one non-interleaved 1F1B window: the per-device batch is cut into ``chunks`` pieces whose
    forward and backward passes interleave across the stages (:meth:`pipeline_step`, which the trainer calls instead of
    strategy + backward; :meth:`pipeline_eval` for validation batches).  The objectives are the token cross-entropies:
    ``seq`` (every position) and ``sft`` (positions of the loss mask, attention inside each packed document; the loss
    is the mean over the trained tokens of the whole per-device batch, whatever the cut into pieces), and the
    sequence-level ones on prepared data: ``dpo`` (a piece holds whole pairs) and ``grpo`` (a piece holds whole response
    groups), for which the last stage scores every piece with the strategy's whole frozen models before the window.
    Gradients accumulate in the flat runtime's fp32 buffers; every parameter lives on exactly one stage, so gradients are
    summed over the data-parallel group only and the gradient norm is summed over the stages.  Checkpoints are put back
    together with the reference's keys: every stage sends its tensors to the first one.

    The transport is point-to-point messages between neighbours (NCCL on GPUs, Gloo on the CPU): there is no fused
    kernel on this path, and on CUDA the last stage computes logits and loss separately (no fused projection + loss)."""

    mode = "pp"

    def __init__(self, grad_accum_steps: int = 1, size: int = 0, chunks: int = 0, comm: str = "nccl", overlap: bool = True,
                 comm_timeout_s: float = 120.0, label_smoothing: float = 0.0, aux_loss_coef: float = 0.0):
        super().__init__(grad_accum_steps, size, "nccl", overlap, comm_timeout_s)
        self.chunks, self.label_smoothing, self.aux_loss_coef = int(chunks), float(label_smoothing), float(aux_loss_coef)
        self._pipe = None
        self._keys: Dict[str, str] = {}

    # -- set-up -------------------------------------------------------------------------------------------------------------
    def _convert(self, model):
        from astrai_b200 import ops
        from astrai_b200.parallel.pipeline import PipelineParallel

        m = self.mesh
        if m.mp_size <= 1:
            raise ValueError("pipeline parallelism needs at least two stages (pp_size >= 2 and as many ranks)")
        if len(model.layers) < m.mp_size:
            raise ValueError(f"{len(model.layers)} decoder layers cannot be cut into {m.mp_size} stages")
        group = m.mp_group if m.mp_group is not None else dist.group.WORLD

        def loss_fn(logits, targets):
            return ops.cross_entropy(logits, targets, label_smoothing=self.label_smoothing)

        self._pipe = PipelineParallel(model, group=group, loss_fn=loss_fn, aux_loss_coef=self.aux_loss_coef)
        stage = self._pipe.stage
        full = {id(v): k for k, v in model.state_dict(keep_vars=True).items()}
        self._keys = {k: full[id(v)] for k, v in stage.state_dict(keep_vars=True).items() if id(v) in full}
        mine = {id(p) for p in stage.parameters()}
        for p in model.parameters():  # what other stages own leaves this rank's memory
            if id(p) not in mine:
                p.data = torch.empty(0, dtype=p.dtype, device=p.device)
        stage.config = model.config
        return stage

    def _is_sharded(self, name, p):
        return True  # every parameter exists on one stage only

    def _averaging_scale(self) -> float:
        return 1.0 / self.mesh.dp_size if (self.use_distributed and self.mesh is not None) else 1.0

    def _unit_backward_done(self, unit):
        pass  # several pieces are in flight per window: units are reduced once, after the window (pipeline_step)

    @property
    def data_parallel_size(self) -> int:
        return self.mesh.dp_size if self.mesh is not None else 1

    @property
    def data_parallel_rank(self) -> int:
        return self.mesh.dp_rank if self.mesh is not None else 0

    # -- one micro-batch of the trainer = one 1F1B window ------------------------------------------------------------------
    def _pieces(self, batch: dict):
        """The batch as the pipeline takes it: ids, targets (masked positions set to the ignored index), the number of
        pieces, per-piece forward keyword arguments and per-piece loss weights."""
        from astrai_b200.trainer.strategy import doc_attention

        unknown = set(batch) - {"input_ids", "target_ids", "position_ids", "loss_mask"}
        if unknown or "target_ids" not in batch:
            raise NotImplementedError("pipeline parallelism trains the token cross-entropy objectives (strategies 'seq' and "
                                      f"'sft'): a batch of input_ids / target_ids [/ position_ids / loss_mask]; got keys {sorted(batch)}")
        stage = self._pipe.stage
        dev = next(stage.parameters()).device
        ids, targets = batch["input_ids"], batch["target_ids"]
        n = ids.shape[0]
        chunks = self.chunks if self.chunks > 0 else min(self.mesh.mp_size, n)
        if n % chunks:
            raise ValueError(f"a per-device batch of {n} cannot be cut into {chunks} pipeline pieces")
        weights = None
        if "loss_mask" in batch:  # the supervised objective: a mean over the trained tokens of the whole batch
            keep = batch["loss_mask"].bool()
            targets = targets.masked_fill(~keep.to(targets.device), -100)
            counts = keep.reshape(chunks, -1).sum(1).double().cpu()  # the loader's batch lives on the host: no device wait
            weights = (counts / counts.sum().clamp(min=1)).tolist()
        kwargs = [{} for _ in range(chunks)]
        if "position_ids" in batch:
            packed = "loss_mask" in batch  # packed documents attend inside themselves, as in the supervised strategy
            for kw, pos in zip(kwargs, batch["position_ids"].chunk(chunks, dim=0)):
                kw["position_ids"] = pos.to(dev)
                if packed:
                    kw["attention"] = doc_attention(pos)
        return ids.to(dev), targets.to(dev), chunks, kwargs, weights

    def _chunks_of(self, n: int, what: str) -> int:
        chunks = self.chunks if self.chunks > 0 else min(self.mesh.mp_size, n)
        if n % chunks:
            raise ValueError(f"a per-device batch of {n} {what} cannot be cut into {chunks} pipeline pieces")
        return chunks

    def _preference_pieces(self, batch: dict, strategy):
        """Preference pairs: a piece is ``m`` chosen answers followed by their ``m`` rejected ones, so that every piece's
        loss is a mean over whole pairs and the window's loss the mean over all of them.  The last stage scores the pieces
        with the frozen reference model first."""
        from astrai_b200.trainer.strategy import dpo_loss, get_logprobs, logprobs_from_logits, padded_causal_attention, reduce_logprobs

        stage = self._pipe.stage
        dev = next(stage.parameters()).device
        n = batch["chosen"].shape[0]
        chunks = self._chunks_of(n, "pairs")
        m = n // chunks
        ids, keep, kwargs, targets = [], [], [], []
        for i in range(chunks):
            rows = slice(i * m, (i + 1) * m)
            piece = torch.cat([batch["chosen"][rows], batch["rejected"][rows]], dim=0)
            mask = torch.cat([batch["chosen_mask"][rows], batch["rejected_mask"][rows]], dim=0)
            attn = padded_causal_attention(piece.ne(0))  # from the host copy
            attn = attn.to(dev) if isinstance(attn, torch.Tensor) else attn
            ids.append(piece.to(dev))
            keep.append(mask.to(dev))
            kwargs.append({"attention": attn})
            if stage.last:
                with torch.no_grad():
                    ref = get_logprobs(strategy.ref_model, ids[-1], attn, keep[-1], strategy.reduction)["logprobs"]
                targets.append({"ids": ids[-1], "keep": keep[-1], "ref": ref})

        def loss_fn(logits, t):
            policy = reduce_logprobs(logprobs_from_logits(logits, t["ids"]), t["keep"], strategy.reduction)
            return dpo_loss(policy, t["ref"], strategy.beta)

        return torch.cat(ids, dim=0), targets, chunks, kwargs, None, loss_fn

    def _group_pieces(self, batch: dict, strategy):
        """Scored response groups: a piece is the groups of ``b / chunks`` prompts; every piece contributes its sums over
        response tokens divided by the batch's token count, so the pieces add up to the batch's loss."""
        from astrai_b200.trainer.strategy import get_logprobs, grpo_terms, logprobs_from_logits, padded_causal_attention, reduce_logprobs

        stage = self._pipe.stage
        dev = next(stage.parameters()).device
        prompts, responses, masks, rewards = batch["prompts"], batch["responses"], batch["masks"], batch["rewards"]
        b, g, rlen = responses.shape
        plen = prompts.shape[1]
        pmask = batch.get("prompt_mask")
        pmask = prompts.ne(0) if pmask is None else pmask
        chunks = self._chunks_of(b, "prompts")
        m = b // chunks
        count = masks.bool().sum().clamp(min=1).float().item()  # the loader's batch lives on the host
        ids, kwargs, targets = [], [], []
        for i in range(chunks):
            rows = slice(i * m, (i + 1) * m)
            prompt = prompts[rows][:, None].expand(-1, g, -1).reshape(m * g, plen)
            valid = torch.cat([pmask[rows][:, None].expand(-1, g, -1).reshape(m * g, plen).bool(), masks[rows].reshape(m * g, rlen).bool()], dim=-1)
            seq = torch.cat([prompt, responses[rows].reshape(m * g, rlen)], dim=-1)
            keep = torch.cat([torch.zeros(m * g, plen, dtype=torch.bool), masks[rows].reshape(m * g, rlen).bool()], dim=-1)
            attn = padded_causal_attention(valid)
            attn = attn.to(dev) if isinstance(attn, torch.Tensor) else attn
            ids.append(seq.to(dev))
            kwargs.append({"attention": attn})
            if stage.last:
                keep_d = keep.to(dev)

                def frozen(model, seq_d=ids[-1], attn=attn, keep_d=keep_d):
                    with torch.no_grad():
                        return get_logprobs(model, seq_d, attn, keep_d, "none")["logprobs"][:, plen - 1:].reshape(m, g, -1)

                targets.append({"ids": ids[-1], "keep": keep_d, "old": frozen(strategy.old_model), "ref": frozen(strategy.ref_model),
                                "rewards": rewards[rows].to(dev), "tok": masks[rows].to(dev).float()})

        def loss_fn(logits, t):
            lp = reduce_logprobs(logprobs_from_logits(logits, t["ids"]), t["keep"], "none")[:, plen - 1:].reshape(m, g, -1)
            surrogate, kl = grpo_terms(lp, t["old"], t["ref"], t["rewards"], t["tok"], strategy.clip_eps)
            return (surrogate + strategy.kl_coef * kl) / count

        return torch.cat(ids, dim=0), targets, chunks, kwargs, [1.0] * chunks, loss_fn

    def pipeline_step(self, model, batch: dict, loss_scale: float, strategy=None) -> dict:
        loss_fn = None
        if "chosen" in batch and "rejected" in batch:
            ids, targets, chunks, kwargs, weights, loss_fn = self._preference_pieces(batch, strategy)
        elif "responses" in batch and "prompts" in batch:
            ids, targets, chunks, kwargs, weights, loss_fn = self._group_pieces(batch, strategy)
        else:
            ids, targets, chunks, kwargs, weights = self._pieces(batch)
        stage = self._pipe.stage
        for u in self.engine.units:
            u.ready = u.reduced = False
        loss = self._pipe.train_step(ids if stage.first else None, targets if stage.last else None, chunks,
                                     micro_shape=(ids.shape[0] // chunks, ids.shape[1]), loss_scale=loss_scale,
                                     micro_kwargs=kwargs, weights=weights, loss_fn=loss_fn)
        if self.gradient_state.sync_gradients:
            for u in reversed(self.engine.units):
                u.ready = True
                self._reduce_unit(u)
            self._finish_reductions()
        return self._shared_loss(loss, ids.device)

    def _shared_loss(self, loss, dev) -> dict:
        """The loss is known on the last stage: hand it to the other stages (logging, validation averages)."""
        from astrai_b200.trainer.strategy import DeferredMetrics

        value = loss.detach().float().reshape(1) if loss is not None else torch.zeros(1, device=dev)
        dist.broadcast(value, src=self.mesh.mp_ranks()[-1], group=self.mesh.mp_group)
        return {"loss": value[0], "metrics": DeferredMetrics(loss=value[0])}

    @torch.no_grad()
    def pipeline_eval(self, model, batch: dict) -> dict:
        """Loss of one batch without gradients (validation): one forward through the stages, piece by piece."""
        from astrai_b200 import ops

        stage = self._pipe.stage
        ids, targets, chunks, kwargs, weights = self._pieces(batch)
        weights = weights or [1.0 / chunks] * chunks
        total = None
        shape = (ids.shape[0] // chunks, ids.shape[1])
        for i, (x, t) in enumerate(zip(ids.chunk(chunks), targets.chunk(chunks))):
            logits = self._pipe.forward_only(x if stage.first else None, micro_shape=shape, **kwargs[i])
            if stage.last:
                piece = ops.cross_entropy(logits, t, label_smoothing=self.label_smoothing) * weights[i]
                total = piece if total is None else total + piece
        return self._shared_loss(total, ids.device)

    # -- state ------------------------------------------------------------------------------------------------------------------
    def _full_state_dict(self, model):
        """Every stage of the first block sends its tensors (under the whole model's keys) to the block's first rank."""
        m = self.mesh
        if m.dp_rank != 0:
            return None
        mine = {self._keys[k]: v.detach().cpu() for k, v in model.state_dict().items() if k in self._keys}
        parts = [None] * m.mp_size if m.mp_rank == 0 else None
        dist.gather_object(mine, parts, dst=m.mp_ranks()[0], group=m.mp_group)
        if parts is None:
            return None
        merged: Dict[str, torch.Tensor] = {}
        for part in parts:
            merged.update(part)
        return merged

    def pack_optimizer_state(self, state):
        """The optimizer state of every stage of the first block, gathered on its first rank (``None`` elsewhere)."""
        m = self.mesh
        if m.dp_rank != 0:
            return None
        parts = [None] * m.mp_size if m.mp_rank == 0 else None
        dist.gather_object(state, parts, dst=m.mp_ranks()[0], group=m.mp_group)
        return {"pipeline_stages": parts} if parts is not None else None

    def unpack_optimizer_state(self, state):
        if isinstance(state, dict) and "pipeline_stages" in state:
            stages = state["pipeline_stages"]
            if len(stages) != self.mesh.mp_size:
                raise RuntimeError(f"the checkpoint holds optimizer state of {len(stages)} pipeline stages, this run has {self.mesh.mp_size}")
            return stages[self.mesh.mp_rank]
        return state
