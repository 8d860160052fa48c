"""Fused FSDP step over NVLink peer memory (``FSDPExecutor(comm="p2p" | "nvls")``).

Per flat unit and optimizer step, instead of ``reduce_scatter`` -> norm pass -> AdamW -> ``all_gather``:

1. ``fsdp_reduce_scatter_``: as soon as the unit's backward pass has finished on the closing micro-batch, ONE kernel
   on the side stream announces "my gradients are ready", waits (bounded) for the same announcement of every peer,
   pulls this rank's shard of the fp32 gradient from all ranks over NVLink (or sums it inside NVSwitch with
   ``multimem.ld_reduce``), writes the reduced shard and adds its squared norm to the clip accumulator.
2. a scalar all-reduce of the squared norm (the only library collective of the step; it is also the point after
   which every rank knows that all peers have finished reading its gradients and using its parameters).
3. ``fsdp_adamw_allgather_``: ONE kernel applies clip x 1/world, AdamW with fp32 moments and master weights on the
   owned shard, stores the new bf16 parameters into EVERY rank's parameter buffer (peer stores or ``multimem.st``)
   and publishes a per-unit "written" flag.  The next forward pass of the unit waits for its peers' flags with a
   one-CTA kernel, so the gather of later units overlaps the compute of earlier ones.

Buffers live in a :class:`~astrai_b200.parallel.symm.SymmetricArena`; the flat parameter and gradient buffers of
the engine are carved from it, so no staging copies exist.  Every device-side wait is bounded (``timeout_s``); a wait
that ran out leaves an error code in the library's status word, which :meth:`FusedFSDP.check` turns into an exception.

The reference delegates all of this to FSDP2 (``astrai/parallel/executor.py:315-428``).
"""

from __future__ import annotations

from typing import Dict, List, Optional

import torch

from astrai_b200.parallel import symm


def arena_bytes_for(model: torch.nn.Module, world_size: int, max_units: int = 512) -> int:
    """Capacity that holds every flat parameter (model dtype) and gradient (fp32) buffer plus flags."""
    total = 0
    n_params = 0
    for p in model.parameters():
        if p.requires_grad:
            total += (p.numel() + 128) * (p.element_size() + 4)
            n_params += 1
    slack = (n_params + 64) * 128 * world_size * 8
    return total + slack + symm.FLAG_KINDS * symm.MAX_RANKS * max_units * 4 + (4 << 20)


class SymmetricAllocator:
    """Allocator handed to :class:`FlatParamEngine`: every flat buffer becomes a sub-buffer of one arena."""

    def __init__(self, arena):
        self.arena = arena
        self._by_ptr: Dict[int, symm.SymmBuffer] = {}

    def alloc(self, numel: int, dtype: torch.dtype, device, what: str) -> torch.Tensor:
        buf = self.arena.alloc(numel, dtype, zero=True)
        self._by_ptr[buf.tensor.data_ptr()] = buf
        return buf.tensor

    def lookup(self, tensor: torch.Tensor) -> symm.SymmBuffer:
        return self._by_ptr[tensor.data_ptr()]


class FusedFSDP:
    MAX_UNITS = 512

    def __init__(self, engine, allocator: SymmetricAllocator, mode: str = "p2p", timeout_s: float = 120.0,
                 max_ctas: int = 64):
        if mode not in ("p2p", "nvls"):
            raise ValueError("mode must be 'p2p' or 'nvls'")
        self.engine, self.alloc, self.arena = engine, allocator, allocator.arena
        self.world, self.rank = engine.world_size, engine.rank
        if mode == "nvls" and not self.arena.has_multicast:
            raise RuntimeError("comm='nvls' needs a multicast-capable symmetric arena (NVSwitch)")
        self.mode, self.timeout_s, self.max_ctas = mode, float(timeout_s), int(max_ctas)
        if len(engine.units) > self.MAX_UNITS:
            raise RuntimeError("too many flat units for the flag array")
        self.flags = self.arena.alloc_flags(self.MAX_UNITS)
        dev = engine.units[0].param_buf.device
        self.sumsq = torch.zeros(1, dtype=torch.float32, device=dev)
        self._index = {u.name: i for i, u in enumerate(engine.units)}
        self._grad = {u.name: allocator.lookup(u.grad_buf) for u in engine.units}
        self._param = {u.name: allocator.lookup(u.param_buf) for u in engine.units}
        self._counter = {u.name: torch.zeros(1, dtype=torch.int32, device=dev) for u in engine.units}
        self._rs_epoch = {u.name: 0 for u in engine.units}
        self._ag_epoch = {u.name: 0 for u in engine.units}
        self._pending: Dict[str, int] = {}
        self.gathers_in_update = True
        for u in engine.units:
            if u.param_buf.dtype != torch.bfloat16:
                raise RuntimeError("the fused FSDP kernels update bf16 parameters (fp32 master weights inside)")
            if u.shard_size % 8:
                raise RuntimeError("shard sizes must be multiples of 8 elements")

    # ------------------------------------------------------------------ step 1: reduce-scatter (+ norm partial)
    def reduce_scatter(self, unit, stream: Optional[torch.cuda.Stream] = None):
        name = unit.name
        self._rs_epoch[name] += 1
        g = self._grad[name]
        mc = g.mc_ptr if self.mode == "nvls" else 0
        args = (g.peer_ptrs, mc, self.flags.peer_ptrs, self.rank, self.rank * unit.shard_size, unit.grad_shard, self.sumsq,
                self._index[name], self.MAX_UNITS, self._rs_epoch[name], self.timeout_s, self.max_ctas)
        if stream is not None:
            stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(stream):
                torch.ops.astrai_b200.fsdp_reduce_scatter_(*args)
        else:
            torch.ops.astrai_b200.fsdp_reduce_scatter_(*args)

    def take_sumsq(self) -> torch.Tensor:
        """Squared norm of this rank's reduced shards since the last call (accumulator is cleared)."""
        out = self.sumsq.clone()
        self.sumsq.zero_()
        return out

    # ------------------------------------------------------------------ step 3: AdamW + all-gather
    def adamw_allgather(self, unit, state: dict, hp: dict, scale: Optional[torch.Tensor]):
        name = unit.name
        self._ag_epoch[name] += 1
        p = self._param[name]
        mc = p.mc_ptr if self.mode == "nvls" else 0
        b1, b2 = hp["betas"]
        torch.ops.astrai_b200.fsdp_adamw_allgather_(
            p.peer_ptrs, mc, self.flags.peer_ptrs, self.rank, self.rank * unit.shard_size, state["master"],
            unit.grad_shard, state["exp_avg"], state["exp_avg_sq"], hp["lr"], b1, b2, hp["eps"], hp["weight_decay"],
            state["step"], scale, self._index[name], self.MAX_UNITS, self._ag_epoch[name], self._counter[name],
            self.max_ctas * 2)
        self._pending[name] = self._ag_epoch[name]

    def wait_params(self, unit):
        """Before the unit's parameters are read again: all peers' shards must have landed."""
        epoch = self._pending.pop(unit.name, None)
        if epoch is None or self.world == 1:
            return
        torch.ops.astrai_b200.comm_wait_flags_(self.flags.tensor, symm.KIND_PARAMS_WRITTEN, self.world, self.rank,
                                               self._index[unit.name], self.MAX_UNITS, epoch, self.timeout_s)

    def wait_all_params(self):
        for u in self.engine.units:
            self.wait_params(u)

    # ------------------------------------------------------------------ failure reporting
    def check(self):
        """Raise if a bounded device-side wait ran out (synchronises with the device)."""
        from astrai_b200.ops import native

        code = native.kernel_status(self.sumsq.device)
        if code in (21, 22, 23):
            torch.ops.astrai_b200.kernel_status_reset(self.sumsq)
            raise RuntimeError(
                f"a peer did not signal within {self.timeout_s:.0f} s (status {code}): a rank is missing, hung or far "
                "behind; the step's gradients / parameters are incomplete")
