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
from astrai_b200.optim.base import OptimizerFactory


@OptimizerFactory.register("fused_adamw")
class FusedAdamW(Optimizer):
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
        else:  # states restored from a checkpoint arrive on the CPU
            for k in ("exp_avg", "exp_avg_sq", "master"):
                if isinstance(st.get(k), torch.Tensor) and st[k].device != p_flat.device:
                    st[k] = st[k].to(p_flat.device)
        return st

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
    def state_dict(self):
        sd = super().state_dict()
        sd["flat_units"] = {
            name: {k: (v.detach().cpu() if isinstance(v, torch.Tensor) else v) for k, v in st.items()}
            for name, st in self._unit_state.items()
        }
        sd["flat_sharded"] = self._sharded
        if self._engine is not None:
            sd["flat_rank"], sd["flat_world"] = self._engine.rank, self._engine.world_size
        return sd

    def load_state_dict(self, state_dict):
        state_dict = dict(state_dict)
        units = state_dict.pop("flat_units", {})
        for k in ("flat_sharded", "flat_rank", "flat_world"):
            state_dict.pop(k, None)
        super().load_state_dict(state_dict)
        for name, st in units.items():
            cur = self._unit_state.get(name)
            if cur is not None:
                for k, v in st.items():
                    if isinstance(v, torch.Tensor) and cur.get(k) is not None:
                        cur[k].copy_(v)
                    else:
                        cur[k] = v
            else:
                self._unit_state[name] = {k: v for k, v in st.items()}
