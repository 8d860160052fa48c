"""AdamW as one kernel per flat buffer.

Plays the role of ``torch.optim.AdamW(fused=True)`` in the reference (``astrai/optim/muon_adamw.py:69-74``,
``scripts/tools/train.py`` optimizer factories) with three differences made for B200 training in bf16:
fp32 moments and (optionally) fp32 master weights whatever the parameter dtype; the gradient is the fp32
``main_grad`` accumulated by the wgrad kernels; the clip coefficient and the data-parallel average arrive as a
device scalar, so no pass over the gradients is spent on scaling.  Under the sharded executor only this rank's
shard of each unit is updated (ZeRO-style partitioned state).

Parameters that are not part of a flat unit (or a plain ``model.parameters()`` list on CPU) take a per-tensor
path with the same math.
"""

from __future__ import annotations

from typing import Any, Dict, Iterable, List, Optional

import torch
from torch.optim import Optimizer

from astrai_b200 import ops
from astrai_b200.optim.base import OptimizerFactory, UntracedOptimizer


@OptimizerFactory.register("fused_adamw")
class FusedAdamW(UntracedOptimizer):
    supports_flat = True
    optimizer_name = "fused_adamw"

    def __init__(self, params, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.01,
                 master_weights: bool = True):
        if isinstance(params, torch.nn.Module):
            params = [p for p in params.parameters() if p.requires_grad]
        super().__init__(params, dict(lr=lr, betas=tuple(betas), eps=eps, weight_decay=weight_decay))
        self.master_weights = master_weights
        self._engine = None
        self._scale: Optional[torch.Tensor] = None
        self._sharded = False
        self._fused = None
        self._unit_state: Dict[str, Dict[str, Any]] = {}
        self.zeroed_in_step = False

    # -- flat binding (called by the executor before every step) --------------------------------------------------
    def bind_flat(self, engine, scale: Optional[torch.Tensor], sharded: bool, fused=None):
        """``fused``: a :class:`~astrai_b200.parallel.fused_fsdp.FusedFSDP`; its kernel then applies the update and
        scatters the new parameters to every rank in the same launch."""
        self._engine, self._scale, self._sharded, self._fused = engine, scale, sharded, fused

    def _unit_buffers(self, unit):
        rank = self._engine.rank if self._sharded else 0
        if self._sharded:
            return unit.param_shard(rank), unit.grad_shard
        return unit.param_buf, unit.grad_buf

    def _state_for(self, unit, p_flat: torch.Tensor):
        st = self._unit_state.get(unit.name)
        if st is None:
            st = {
                "step": 0,
                "exp_avg": torch.zeros(p_flat.numel(), dtype=torch.float32, device=p_flat.device),
                "exp_avg_sq": torch.zeros(p_flat.numel(), dtype=torch.float32, device=p_flat.device),
                "master": p_flat.float().clone() if (self.master_weights and p_flat.dtype != torch.float32) else None,
            }
            self._unit_state[unit.name] = st
        elif "_layout" in st:
            self._localize(unit, st, p_flat)
        return st

    def _localize(self, unit, st: Dict[str, Any], p_flat: torch.Tensor):
        """Turn a unit state that came out of a checkpoint into this rank's working state.

        ``full`` layout: tensors cover the whole unit (written by an unsharded run, or gathered from every rank by
        :meth:`state_dict`); a sharded run cuts its own ``[rank*S, (rank+1)*S)`` range out of it, after padding or
        trimming the tail to this run's unit size (the padding of a unit depends on the world size).
        ``shard`` layout: tensors are one rank's shard and are only valid for that rank of a run of that world size.
        """
        layout, saved = st.pop("_layout"), st.pop("_saved", (None, None))
        eng = self._engine
        world = eng.world_size if (eng is not None and self._sharded) else 1
        rank = eng.rank if (eng is not None and self._sharded) else 0
        n = p_flat.numel()
        for k in ("exp_avg", "exp_avg_sq", "master"):
            v = st.get(k)
            if not isinstance(v, torch.Tensor):
                continue
            v = v.reshape(-1)
            if layout == "full":
                total = n * world
                if v.numel() < total:
                    v = torch.nn.functional.pad(v, (0, total - v.numel()))
                v = v[rank * n:(rank + 1) * n] if world > 1 else v[:total]
            else:
                if tuple(saved) != (rank, world):
                    raise RuntimeError(
                        f"optimizer state of unit {unit.name} is shard {saved[0]} of {saved[1]} ranks, but this process is "
                        f"rank {rank} of {world}: a per-rank optimizer file can only be loaded by the rank that wrote it")
                if v.numel() != n:
                    raise RuntimeError(f"optimizer shard of unit {unit.name} has {v.numel()} elements, expected {n}")
            st[k] = v.to(device=p_flat.device, dtype=torch.float32, copy=True).contiguous()
        if self.master_weights and p_flat.dtype != torch.float32 and st.get("master") is None:
            st["master"] = p_flat.float().clone()

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        done_units = set()
        for group in self.param_groups:
            hp = dict(lr=group["lr"], betas=group["betas"], eps=group["eps"], weight_decay=group["weight_decay"])
            loose: List[torch.nn.Parameter] = []
            group_ids = {id(p) for p in group["params"]}
            for p in group["params"]:
                unit = getattr(p, "_flat_unit", None) if self._engine is not None else None
                if unit is None:
                    loose.append(p)
                    continue
                if unit.name in done_units:
                    continue
                if not all(id(q) in group_ids for q in unit.params):
                    raise ValueError(f"unit {unit.name} spans several param groups; keep a unit's parameters together")
                done_units.add(unit.name)
                p_flat, g_flat = self._unit_buffers(unit)
                st = self._state_for(unit, p_flat)
                st["step"] += 1
                if self._fused is not None and self._sharded:
                    self._fused.adamw_allgather(unit, st, hp, self._scale)
                    continue
                ops.adamw_(p_flat, g_flat, st["exp_avg"], st["exp_avg_sq"], step=st["step"], master=st["master"],
                           grad_scale=self._scale, zero_grad=False, **hp)
            for p in loose:
                self._step_tensor(p, hp)
        self._scale = None
        return loss

    def _step_tensor(self, p, hp):
        grad = getattr(p, "main_grad", None)
        if grad is None:
            if p.grad is None:
                return
            grad = p.grad.float()
        st = self.state[p]
        if not st:
            st["step"] = 0
            st["exp_avg"] = torch.zeros(p.numel(), dtype=torch.float32, device=p.device)
            st["exp_avg_sq"] = torch.zeros(p.numel(), dtype=torch.float32, device=p.device)
            st["master"] = p.detach().float().reshape(-1).clone() if (self.master_weights and p.dtype != torch.float32) else None
        st["step"] += 1
        flat_p = p.data.view(-1) if p.data.is_contiguous() else None
        target = flat_p if flat_p is not None else p.data.reshape(-1).clone()
        ops.adamw_(target, grad.reshape(-1).contiguous(), st["exp_avg"], st["exp_avg_sq"], step=st["step"],
                   master=st["master"], grad_scale=self._scale, zero_grad=False, **hp)
        if flat_p is None:
            p.data.copy_(target.view_as(p))

    def zero_grad(self, set_to_none: bool = True):
        if self._engine is not None:
            self._engine.zero_grad()
        super().zero_grad(set_to_none=set_to_none)

    # -- (de)serialisation: unit states are stored under their unit names -------------------------------------------
    def _gathered(self, v: torch.Tensor, world: int) -> Optional[torch.Tensor]:
        """Every rank's shard of one state tensor, concatenated in rank order (collective); kept on rank 0 only."""
        import torch.distributed as dist

        full = torch.empty(world * v.numel(), dtype=v.dtype, device=v.device)
        dist.all_gather_into_tensor(full, v.contiguous())
        return full.cpu() if dist.get_rank() == 0 else None

    def state_dict(self, gather: bool = True):
        """Optimizer state with the flat unit states under ``flat_units``.

        Under the sharded executor on more than one rank this is a COLLECTIVE when ``gather`` is true: the moments
        and master weights of every unit are all-gathered so that rank 0's dict holds whole units (``flat_layout =
        "full"``), which any rank of any world size can load.  ``gather=False`` never communicates and returns this
        rank's shards (``flat_layout = "shard"``, tagged with rank and world size) - the form used for an emergency
        save while a peer is down, to be written to a per-rank file.  The reference saves rank 0's shard only and
        cannot resume it on the other ranks (``astrai/parallel/executor.py:135-136``).
        """
        import torch.distributed as dist

        sd = super().state_dict()
        eng = self._engine
        world = eng.world_size if eng is not None else 1
        multi = self._sharded and world > 1 and dist.is_available() and dist.is_initialized()
        units = {}
        for name, st in self._unit_state.items():
            entry = {}
            pending = "_layout" in st  # restored and not used yet: pass it through unchanged
            for k, v in st.items():
                if isinstance(v, torch.Tensor):
                    v = self._gathered(v.detach(), world) if (multi and gather and not pending) else v.detach().cpu()
                entry[k] = v
            units[name] = entry
        sd["flat_units"] = units
        sd["flat_sharded"] = self._sharded
        sd["flat_layout"] = "full" if (not multi or gather) else "shard"
        if eng is not None:
            sd["flat_rank"], sd["flat_world"] = eng.rank, eng.world_size
        return sd

    def load_state_dict(self, state_dict):
        state_dict = dict(state_dict)
        units = state_dict.pop("flat_units", {})
        sharded = state_dict.pop("flat_sharded", False)
        saved = (state_dict.pop("flat_rank", 0), state_dict.pop("flat_world", 1))
        layout = state_dict.pop("flat_layout", None)
        if layout is None:  # files written before the layout tag existed
            layout = "shard" if (sharded and saved[1] > 1) else "full"
        super().load_state_dict(state_dict)
        for name, st in units.items():
            if st.get("_layout") is not None:  # a pass-through entry keeps its own tags
                self._unit_state[name] = dict(st)
                continue
            entry = dict(st)
            entry["_layout"], entry["_saved"] = layout, saved
            self._unit_state[name] = entry
