"""Full-shard residency for the flat FSDP runtime: parameters and gradients exist whole only while a unit computes.

At rest a rank holds, per flat unit, its own bf16 parameter shard, its fp32 gradient-shard accumulator and the optimizer
state of that shard - ``1 / world`` of everything.  The unit's full parameter buffer and full fp32 gradient buffer keep
their tensors (every ``Parameter.data`` and ``main_grad`` is a view of them) but their *storage* is released
(``resize_(0)``) and re-created when the unit is about to compute:

* forward: a pre-hook re-creates the parameter storage and all-gathers the shards into it (on the side stream; the gather
  of the next unit is issued before this unit's compute, so it runs under it); a forward hook releases the storage of
  decoder blocks again (``reshard_after_forward``), units outside the block list (embedding, final norm, head) stay
  resident until the backward pass has finished with them;
* backward: a hook on the unit's outputs re-gathers the parameters (prefetching the unit before it) and creates a zeroed
  gradient buffer; when the gradient of the unit's input has been produced, the gradient buffer is reduce-scattered, the
  result is added to the rank's fp32 shard accumulator, and both storages are released.  This happens in EVERY
  micro-batch (a full gradient buffer does not survive the unit's backward pass), so an accumulation window of ``k``
  micro-batches moves ``k`` times the gradient bytes of the replicated mode - the price of the memory;
* optimizer step: AdamW reads the accumulator and writes the rank's parameter shard; nothing is gathered until the next
  forward pass needs it.

The all-gather writes into a buffer whose views autograd has saved for the backward pass; it runs under
``torch.autograd._unsafe_preserve_version_counter`` because it re-creates the values that were saved (same shards, no
update in between).

Counterpart in the reference: ``fully_shard`` per decoder block with ``reshard_after_forward``
(``astrai/parallel/executor.py:338-361``); here the unit is the flat buffer and the collectives move whole units.
"""

from __future__ import annotations

import contextlib
from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from astrai_b200.parallel.flat import FlatParamEngine, FlatUnit


def _nbytes(t: torch.Tensor) -> int:
    return t.numel() * t.element_size()


class ReshardRuntime:
    def __init__(self, engine: FlatParamEngine, comm_stream=None, group=None, reshard_after_forward: bool = True):
        self.engine, self.stream, self.group = engine, comm_stream, group
        self.reshard_after_forward = reshard_after_forward
        self.order: Dict[str, int] = {u.name: i for i, u in enumerate(engine.units)}
        self.transient = {u.name: self._is_block(u) for u in engine.units}
        self._params_in: Dict[str, bool] = {}
        self._grads_in: Dict[str, bool] = {}
        self._events: Dict[str, object] = {}
        self._bwd_seen: Dict[str, bool] = {}
        self.peak_resident_params = 0  # largest number of units whose parameters were whole at the same time
        rank = engine.rank
        dev = engine.units[0].param_buf.device
        # one scratch for every unit's reduce-scatter result: the reductions are ordered on one stream
        self._rs_out = torch.empty(max(u.shard_size for u in engine.units), dtype=torch.float32, device=dev)
        for u in engine.units:
            a, b = u.shard_range(rank)
            u.local_shard = u.param_buf[a:b].clone()
            u.grad_shard = torch.zeros(u.shard_size, dtype=torch.float32, device=u.param_buf.device)
            self._params_in[u.name] = self._grads_in[u.name] = True
            self.release(u)

    @staticmethod
    def _is_block(unit: FlatUnit) -> bool:
        """Units made of elements of a module list (decoder blocks): the ones that are released between their forward
        and backward passes."""
        return all(name.rsplit(".", 1)[-1].isdigit() for name in unit.module_names)

    # -- residency ---------------------------------------------------------------------------------------------------
    def params_resident(self, unit: FlatUnit) -> bool:
        return self._params_in[unit.name]

    def resident_bytes(self) -> int:
        return sum(u.param_buf.untyped_storage().size() + u.grad_buf.untyped_storage().size() for u in self.engine.units)

    def _side(self):
        return torch.cuda.stream(self.stream) if self.stream is not None else contextlib.nullcontext()

    def _issue_gather(self, unit: FlatUnit):
        if self._params_in[unit.name]:
            return
        unit.param_buf.untyped_storage().resize_(_nbytes(unit.param_buf))
        self._params_in[unit.name] = True
        self.peak_resident_params = max(self.peak_resident_params, sum(self._params_in.values()))
        if self.stream is not None:
            self.stream.wait_stream(torch.cuda.current_stream())  # earlier users of the recycled memory come first
        with self._side(), torch.autograd._unsafe_preserve_version_counter(unit.param_buf), torch.no_grad():
            if self.engine.world_size > 1:
                dist.all_gather_into_tensor(unit.param_buf, unit.local_shard, group=self.group)
            else:
                unit.param_buf.copy_(unit.local_shard)
            if self.stream is not None:
                ev = torch.cuda.Event()
                ev.record(self.stream)
                self._events[unit.name] = ev

    def unshard(self, unit: FlatUnit, prefetch: Optional[int] = None):
        """Make ``unit``'s parameters whole on the current stream; ``prefetch`` = +1 / -1 also starts the gather of the
        unit after / before it."""
        self._issue_gather(unit)
        ev = self._events.pop(unit.name, None)
        if ev is not None:
            torch.cuda.current_stream().wait_event(ev)
        if prefetch:
            j = self.order[unit.name] + prefetch
            if 0 <= j < len(self.engine.units):
                self._issue_gather(self.engine.units[j])

    def ensure_grads(self, unit: FlatUnit):
        if self._grads_in[unit.name]:
            return
        unit.grad_buf.untyped_storage().resize_(_nbytes(unit.grad_buf))
        unit.grad_buf.zero_()
        self._grads_in[unit.name] = True

    def release_params(self, unit: FlatUnit):
        if self._params_in[unit.name]:
            ev = self._events.pop(unit.name, None)
            if ev is not None:  # gathered ahead of time and never used: the gather must not outlive the memory
                torch.cuda.current_stream().wait_event(ev)
            unit.param_buf.untyped_storage().resize_(0)
            self._params_in[unit.name] = False

    def release(self, unit: FlatUnit):
        self.release_params(unit)
        if self._grads_in[unit.name]:
            unit.grad_buf.untyped_storage().resize_(0)
            self._grads_in[unit.name] = False

    def release_all(self):
        for u in self.engine.units:
            self.release(u)

    def unshard_all(self):
        for u in self.engine.units:
            self.unshard(u)

    # -- hooks ---------------------------------------------------------------------------------------------------------
    def before_forward(self, unit: FlatUnit):
        self.unshard(unit, prefetch=+1 if self.transient[unit.name] else None)
        if torch.is_grad_enabled() and not self.transient[unit.name]:
            self.ensure_grads(unit)  # units outside the block list get no output hook: their buffer exists from first use

    def after_forward(self, unit: FlatUnit, output):
        """Forward hook of a block: release the parameters, and arrange for them to be back before the block's backward."""
        if not self.transient[unit.name]:
            return
        if torch.is_grad_enabled():
            tensors: List[torch.Tensor] = []
            self._collect(output, tensors)
            for t in tensors:
                t.register_hook(lambda g, u=unit: self.before_backward(u))
        if self.reshard_after_forward:
            self.release_params(unit)

    def _collect(self, obj, out: List[torch.Tensor]):
        if isinstance(obj, torch.Tensor):
            if obj.requires_grad:
                out.append(obj)
        elif isinstance(obj, dict):
            for v in obj.values():
                self._collect(v, out)
        elif isinstance(obj, (list, tuple)):
            for v in obj:
                self._collect(v, out)

    def begin_backward(self):
        self._bwd_seen = {}

    def before_backward(self, unit: FlatUnit):
        if self._bwd_seen.get(unit.name):
            return None
        self._bwd_seen[unit.name] = True
        self.unshard(unit, prefetch=-1)
        self.ensure_grads(unit)
        return None

    def reduce(self, unit: FlatUnit):
        """Reduce-scatter the unit's gradient buffer, add the result to the shard accumulator, release both storages."""
        if not self._grads_in[unit.name]:
            self.release_params(unit)
            return
        if self.stream is not None:
            self.stream.wait_stream(torch.cuda.current_stream())
        with self._side(), torch.no_grad():
            if self.engine.world_size > 1:
                out = self._rs_out[: unit.shard_size]
                dist.reduce_scatter_tensor(out, unit.grad_buf, group=self.group)
                unit.grad_shard.add_(out)
            else:
                unit.grad_shard.add_(unit.grad_buf[: unit.shard_size])
        if self.stream is not None:
            unit.grad_buf.record_stream(self.stream)  # the side stream still reads it: defer the reuse of its memory
        self.release(unit)

    def finish(self):
        if self.stream is not None:
            torch.cuda.current_stream().wait_stream(self.stream)

    def zero_accumulators(self):
        for u in self.engine.units:
            u.grad_shard.zero_()
