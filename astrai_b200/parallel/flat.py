"""Flat parameter / gradient buffers: the memory layout behind the DDP and FSDP executors.

Every *unit* (one decoder block, the embedding, the final norm + head) owns
  * one contiguous bf16 (or fp32) buffer holding all of its parameters - each ``Parameter.data`` is re-pointed to a
    view of it, q/k/v and gate/up laid out back to back so that they run as ONE tcgen05 GEMM, and
  * one contiguous fp32 gradient buffer; every parameter gets a ``main_grad`` view into which the wgrad kernels
    accumulate directly (``D += dY^T X`` in the GEMM epilogue), so there are no per-parameter ``.grad`` tensors,
    no bf16 gradient round trip and no separate accumulation pass over micro-batches.
Units are padded to a multiple of ``world_size * 128`` elements so a unit splits into equal, 256-byte aligned
shards: rank ``r`` owns elements ``[r*S, (r+1)*S)`` of the unit for the sharded optimizer state (FSDP) and one
collective (all-reduce, reduce-scatter, all-gather) moves a whole unit.

This replaces FSDP2's per-parameter DTensor sharding and DDP's 25 MB buckets of the reference
(``astrai/parallel/executor.py:254-428``) with a layout sized for 180 GB of HBM3e and NVSwitch collectives.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional

import torch
import torch.nn as nn

ALIGN = 128  # elements; 256 B for bf16, 512 B for fp32


@dataclass
class FlatUnit:
    name: str
    module_names: List[str]
    params: List[nn.Parameter] = field(default_factory=list)
    param_names: List[str] = field(default_factory=list)
    offsets: List[int] = field(default_factory=list)
    numel: int = 0  # padded
    param_buf: Optional[torch.Tensor] = None
    grad_buf: Optional[torch.Tensor] = None
    shard_size: int = 0
    grad_shard: Optional[torch.Tensor] = None  # fp32 [shard_size]: reduce-scatter result (sharded modes)
    local_shard: Optional[torch.Tensor] = None  # this rank's parameter shard when the full buffer is released at rest
    ready: bool = False  # gradient of the current step fully accumulated
    reduced: bool = False
    tag: str = ""  # set when an executor splits units by parameter kind (replicated / sharded): picks the reduce group

    def shard_range(self, rank: int):
        return rank * self.shard_size, (rank + 1) * self.shard_size

    def param_shard(self, rank: int) -> torch.Tensor:
        if self.local_shard is not None:
            return self.local_shard
        a, b = self.shard_range(rank)
        return self.param_buf[a:b]

    def segments(self, lo: int, hi: int):
        """(param index, start in param, start in [lo,hi) window, length) for the params overlapping [lo, hi)."""
        out = []
        for i, (off, p) in enumerate(zip(self.offsets, self.params)):
            a, b = max(off, lo), min(off + p.numel(), hi)
            if a < b:
                out.append((i, a - off, a - lo, b - a))
        return out


def _fold_autograd_grad(p: nn.Parameter):
    """A gradient that reached the parameter through autograd (an op without a wgrad kernel: stacked expert weights,
    LoRA factors, biases, every op on the CPU path) is added to ``main_grad`` at once and dropped, so that the flat
    buffers stay the single place where gradients live.  The native wgrad kernels return ``None`` to autograd and
    never come through here."""
    if p.grad is not None:
        p.main_grad.add_(p.grad.to(p.main_grad.dtype).view_as(p.main_grad))
        p.grad = None


def _ordered_params(module: nn.Module, prefix: str):
    """named_parameters with q,k,v and gate,up made adjacent (fusable) inside attention / MLP modules."""
    seen = set()
    out = []

    def visit(mod: nn.Module, pfx: str):
        names = list(mod._modules.keys())
        pref = []
        if all(n in mod._modules for n in ("q_proj", "k_proj", "v_proj")):
            pref = ["q_proj", "k_proj", "v_proj"]
        elif all(n in mod._modules for n in ("gate", "up", "down")):
            pref = ["gate", "up"]
        order = pref + [n for n in names if n not in pref]
        for pname, p in mod._parameters.items():
            if p is not None and id(p) not in seen:
                seen.add(id(p))
                out.append((pfx + pname, p))
        for n in order:
            child = mod._modules[n]
            if child is not None:
                visit(child, pfx + n + ".")

    visit(module, prefix)
    return out


def default_units(model: nn.Module) -> List[List[str]]:
    """One unit per element of every ``ModuleList`` child, one for each other direct child with parameters."""
    groups: List[List[str]] = []
    for name, child in model.named_children():
        if isinstance(child, nn.ModuleList):
            groups.extend([[f"{name}.{i}"] for i in range(len(child))])
        elif any(True for _ in child.parameters()):
            groups.append([name])
    return groups


class FlatParamEngine:
    """Builds the units for a model and keeps the bookkeeping the executors need."""

    def __init__(self, model: nn.Module, world_size: int = 1, rank: int = 0, grad_dtype=torch.float32,
                 units: Optional[List[List[str]]] = None, allocator: Optional[Callable] = None,
                 tag_fn: Optional[Callable[[str, nn.Parameter], str]] = None):
        """``tag_fn(name, param)``: when given, every unit is split into one unit per tag (``<unit>#<tag>``), so that
        parameters whose gradients are reduced over different process groups never share a flat buffer."""
        self.model = model
        self.world_size, self.rank = world_size, rank
        self.grad_dtype = grad_dtype
        self.units: List[FlatUnit] = []
        self._alloc = allocator or (lambda n, dtype, device, what: torch.zeros(n, dtype=dtype, device=device))
        claimed = set()
        for names in (units or default_units(model)):
            by_tag: Dict[str, FlatUnit] = {}
            for mname in names:
                mod = model.get_submodule(mname)
                for pname, p in _ordered_params(mod, mname + "."):
                    if id(p) in claimed or not p.requires_grad:
                        continue
                    claimed.add(id(p))
                    tag = tag_fn(pname, p) if tag_fn is not None else ""
                    unit = by_tag.get(tag)
                    if unit is None:
                        base = "+".join(names)
                        unit = by_tag[tag] = FlatUnit(name=f"{base}#{tag}" if tag else base, module_names=list(names), tag=tag)
                    unit.params.append(p)
                    unit.param_names.append(pname)
            for unit in by_tag.values():
                self._layout(unit)
                self.units.append(unit)
        self._install_fused_views()

    # ------------------------------------------------------------------ layout
    def _layout(self, unit: FlatUnit):
        dtype, device = unit.params[0].dtype, unit.params[0].device
        if any(p.dtype != dtype for p in unit.params):
            raise ValueError(f"unit {unit.name}: mixed parameter dtypes")
        off = 0
        for p in unit.params:
            unit.offsets.append(off)
            off += -(-p.numel() // ALIGN) * ALIGN
        quantum = ALIGN * self.world_size
        unit.numel = -(-off // quantum) * quantum
        unit.shard_size = unit.numel // self.world_size
        unit.param_buf = self._alloc(unit.numel, dtype, device, "param")
        unit.grad_buf = self._alloc(unit.numel, self.grad_dtype, device, "grad")
        with torch.no_grad():
            for p, o in zip(unit.params, unit.offsets):
                view = unit.param_buf[o:o + p.numel()].view(p.shape)
                view.copy_(p.data)
                p.data = view
                p.main_grad = unit.grad_buf[o:o + p.numel()].view(p.shape)
                p._flat_unit = unit
                p.grad = None
                p.register_post_accumulate_grad_hook(_fold_autograd_grad)

    def _fuse(self, unit: FlatUnit, parts: List[nn.Parameter]):
        """A [sum(rows), cols] view over adjacent 2-D parameters (None if they are not back to back)."""
        idx = []
        for p in parts:
            where = [i for i, q in enumerate(unit.params) if q is p]
            if not where:
                return None
            idx.append(where[0])
        cols = parts[0].shape[1]
        start = unit.offsets[idx[0]]
        expect = start
        for i, p in zip(idx, parts):
            if unit.offsets[i] != expect or p.dim() != 2 or p.shape[1] != cols:
                return None
            expect += p.numel()
        rows = sum(p.shape[0] for p in parts)
        view = unit.param_buf[start:start + rows * cols].view(rows, cols)
        view.main_grad = unit.grad_buf[start:start + rows * cols].view(rows, cols)
        return view

    def _install_fused_views(self):
        owner: Dict[int, FlatUnit] = {id(p): u for u in self.units for p in u.params}

        def plain(mod, names):
            return all(type(getattr(mod, n, None)).__name__ == "Linear" for n in names)

        for mod in self.model.modules():  # any attention / MLP block that declares the slot (the tensor-parallel ones too)
            if hasattr(mod, "fused_qkv") and plain(mod, ("q_proj", "k_proj", "v_proj")):
                parts = [mod.q_proj.weight, mod.k_proj.weight, mod.v_proj.weight]
                unit = owner.get(id(parts[0]))
                mod.fused_qkv = self._fuse(unit, parts) if unit is not None else None
            elif hasattr(mod, "fused_gate_up") and plain(mod, ("gate", "up")):
                parts = [mod.gate.weight, mod.up.weight]
                unit = owner.get(id(parts[0]))
                mod.fused_gate_up = self._fuse(unit, parts) if unit is not None else None

    # ------------------------------------------------------------------ helpers
    def zero_grad(self):
        for u in self.units:
            u.grad_buf.zero_()
            u.ready = u.reduced = False

    def grad_sumsq(self, sharded: bool = False) -> torch.Tensor:
        from astrai_b200 import ops

        dev = self.units[0].grad_buf.device
        acc = torch.zeros(1, dtype=torch.float32, device=dev)
        for u in self.units:
            ops.sumsq(u.grad_shard if sharded else u.grad_buf, acc)
        return acc

    def unit_of(self, p: nn.Parameter) -> Optional[FlatUnit]:
        return getattr(p, "_flat_unit", None)

    def total_numel(self) -> int:
        return sum(u.numel for u in self.units)

    def materialize_grads(self, scale: Optional[torch.Tensor] = None):
        """Give optimizers that only know ``p.grad`` a gradient in the parameter dtype (copy of ``main_grad``)."""
        for u in self.units:
            for p in u.params:
                g = p.main_grad if scale is None else p.main_grad * scale
                p.grad = g.to(p.dtype)

    def drop_grads(self):
        for u in self.units:
            for p in u.params:
                p.grad = None
