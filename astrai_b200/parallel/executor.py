"""Training executors: parallel strategy + gradient accumulation behind one interface.

Interface of the reference (``astrai/parallel/executor.py:160-247``): ``prepare``, ``accumulate``, ``backward``,
``clip_grad_norm``, ``checkpoint_context``, ``unwrap_model``, ``sync_gradients``, ``grad_accum_steps``.
Modes ``none``, ``ddp``, ``fsdp`` exist in the reference as wrappers over torch DDP / FSDP2; here each has

* ``impl="flat"`` (default on CUDA): this framework's own runtime over :class:`FlatParamEngine` - wgrad kernels
  accumulate into fp32 flat buffers, one collective per unit on a side stream overlapped with the rest of the
  backward pass, clip coefficient kept on the device and folded into the fused AdamW kernel, sharded fp32
  optimizer state for FSDP, parameter all-gather overlapped with the next forward pass;
* ``impl="torch"``: ``DistributedDataParallel`` / ``fully_shard`` wrappers with the reference's semantics, used on
  CPU (Gloo) and as the comparison baseline.
"""

from __future__ import annotations

import contextlib
import logging
import os
from contextlib import contextmanager
from typing import Any, Callable, Dict, List, Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn

from astrai_b200.factory import BaseFactory
from astrai_b200.parallel.flat import FlatParamEngine, FlatUnit
from astrai_b200.parallel.setup import get_rank, get_world_size

logger = logging.getLogger(__name__)


# --------------------------------------------------------------------------- state-dict broadcast / frozen copies
def broadcast_state_dict(state_dict: Optional[Dict[str, torch.Tensor]], src: int = 0) -> Optional[Dict[str, torch.Tensor]]:
    """Send a state dict from ``src`` to every rank (collective).  Tensors stay on the device they are on."""
    if not dist.is_initialized() or dist.get_world_size() == 1:
        return state_dict
    me = dist.get_rank()
    header = [None]
    if me == src:
        header[0] = [(k, tuple(v.shape), v.dtype, str(v.device)) for k, v in state_dict.items()]
    dist.broadcast_object_list(header, src=src)
    if me != src:
        local_dev = os.environ.get("LOCAL_DEVICE")
        state_dict = {}
        for k, shape, dtype, dev in header[0]:
            target = torch.device(dev)
            if target.type == "cuda" and local_dev:
                target = torch.device(local_dev)
            state_dict[k] = torch.empty(shape, dtype=dtype, device=target)
    for t in state_dict.values():
        dist.broadcast(t, src=src)
    return state_dict


def create_ref_model(model_fn: Callable[[], nn.Module], executor: Optional["BaseExecutor"] = None,
                     model: Optional[nn.Module] = None, state_dict: Optional[Dict[str, torch.Tensor]] = None,
                     device: Optional[str] = None) -> Optional[nn.Module]:
    """A frozen, eval-mode copy of the current weights (reference / behaviour policy for DPO and GRPO)."""
    if state_dict is None and executor is not None and model is not None:
        state_dict = executor.unwrap_model(model)
    if executor is not None and executor.use_distributed:
        state_dict = broadcast_state_dict(state_dict)
    if state_dict is None:
        return None
    ref = model_fn()
    first = next(iter(state_dict.values()))
    if first.is_floating_point():
        ref = ref.to(first.dtype)
    ref.load_state_dict(state_dict)
    ref.requires_grad_(False)
    ref.eval()
    return ref.to(device=device) if device is not None else ref


# --------------------------------------------------------------------------- accumulation gating
class GradientState:
    def __init__(self, grad_accum_steps: int = 1):
        self.num_steps = max(int(grad_accum_steps), 1)
        self._step = 0
        self._sync_gradients = True

    @property
    def sync_gradients(self) -> bool:
        return self._sync_gradients

    def _do_sync(self):
        self._step += 1
        self._sync_gradients = self._step % self.num_steps == 0


class AccumOptimizer:
    """Lets ``step`` / ``zero_grad`` through only on the micro-batch that closes an accumulation window."""

    def __init__(self, optimizer, gradient_state: GradientState, executor: Optional["BaseExecutor"] = None):
        self.optimizer, self.gradient_state, self.executor = optimizer, gradient_state, executor

    def step(self, closure=None):
        if not self.gradient_state.sync_gradients:
            return
        if self.executor is not None:
            self.executor._before_optimizer_step(self.optimizer)
        self.optimizer.step(closure)
        if self.executor is not None:
            self.executor._after_optimizer_step(self.optimizer)

    def zero_grad(self):
        if not self.gradient_state.sync_gradients:
            return
        if self.executor is not None and self.executor._zero_grad(self.optimizer):
            return
        self.optimizer.zero_grad()

    @property
    def param_groups(self):
        return self.optimizer.param_groups

    def state_dict(self, gather: bool = True):
        """``gather=False`` asks a sharded optimizer for its local shard only (no communication).  Executors whose ranks
        hold different parameters (pipeline stages) put the ranks' states together (``pack_optimizer_state``)."""
        if not gather:
            try:
                return self.optimizer.state_dict(gather=False)
            except TypeError:
                pass
        state = self.optimizer.state_dict()
        pack = getattr(self.executor, "pack_optimizer_state", None)
        return pack(state) if pack is not None else state

    def load_state_dict(self, d):
        unpack = getattr(self.executor, "unpack_optimizer_state", None)
        self.optimizer.load_state_dict(unpack(d) if unpack is not None else d)


class AccumScheduler:
    def __init__(self, scheduler, gradient_state: GradientState):
        self.scheduler, self.gradient_state = scheduler, gradient_state

    def step(self):
        if self.gradient_state.sync_gradients:
            self.scheduler.step()

    def state_dict(self):
        return self.scheduler.state_dict()

    def load_state_dict(self, d):
        self.scheduler.load_state_dict(d)

    def get_last_lr(self):
        return self.scheduler.get_last_lr()


# --------------------------------------------------------------------------- base
class BaseExecutor:
    flat_capable = False

    def __init__(self, grad_accum_steps: int = 1):
        self.gradient_state = GradientState(grad_accum_steps)
        self.engine: Optional[FlatParamEngine] = None

    # -- construction -----------------------------------------------------------------------------------------
    def prepare(self, model_fn, optimizer_fn=None, scheduler_fn=None, before_wrap=None, after_wrap=None):
        model = model_fn()
        if before_wrap is not None:
            model = before_wrap(model)
        model = self._prepare_model(model)
        if after_wrap is not None:
            model = after_wrap(model)
        optimizer = scheduler = None
        if optimizer_fn is not None:
            raw = optimizer_fn(model)
            if scheduler_fn is not None:
                scheduler = AccumScheduler(scheduler_fn(raw), self.gradient_state)
            optimizer = AccumOptimizer(raw, self.gradient_state, self)
        return model, optimizer, scheduler

    def _prepare_model(self, model: nn.Module) -> nn.Module:
        return model

    # -- accumulation / backward --------------------------------------------------------------------------------
    def _no_sync(self, model: nn.Module):
        return contextlib.nullcontext()

    @contextmanager
    def accumulate(self, model: nn.Module):
        self.gradient_state._do_sync()
        if self.gradient_state.sync_gradients:
            yield
        else:
            with self._no_sync(model):
                yield

    def backward(self, loss: torch.Tensor, gradient: Optional[torch.Tensor] = None):
        loss.backward(gradient)

    # -- optimizer-step plumbing (overridden by the flat runtime) -------------------------------------------------
    def _before_optimizer_step(self, optimizer):
        pass

    def _after_optimizer_step(self, optimizer):
        pass

    def _zero_grad(self, optimizer) -> bool:
        return False

    # -- state --------------------------------------------------------------------------------------------------
    def unwrap_model(self, model: nn.Module):
        return model.state_dict()

    def local_state_dict(self, model: nn.Module):
        """The full model state from this rank's memory alone, without any communication, or ``None`` when the
        parameters are sharded at rest.  Used for an emergency save while a peer is down."""
        inner = getattr(model, "module", model)
        return inner.state_dict()

    communicates_every_micro_batch = False  # model-parallel executors set this: every forward pass has collectives

    def before_param_use(self, p) -> None:
        """Called by code that reads a parameter without calling the module that owns it (the fused projection + loss
        reads ``lm_head.weight`` directly): makes the parameter's pending gather visible to the current stream."""

    def _gather_state_dict(self, model: nn.Module):
        sd = self.unwrap_model(model)
        return None if (self.use_distributed and get_rank() != 0) else sd

    @contextmanager
    def checkpoint_context(self, model: nn.Module):
        if self.use_distributed:
            dist.barrier()
        yield self._gather_state_dict(model)
        if self.use_distributed:
            dist.barrier()

    @property
    def use_distributed(self) -> bool:
        return get_world_size() > 1

    @property
    def sync_gradients(self) -> bool:
        return self.gradient_state.sync_gradients

    @property
    def grad_accum_steps(self) -> int:
        return self.gradient_state.num_steps

    def clip_grad_norm(self, model: nn.Module, max_norm: float) -> float:
        total = torch.nn.utils.clip_grad_norm_(model.parameters(), max_norm)
        return total.item() if isinstance(total, torch.Tensor) else float(total)


class ExecutorFactory(BaseFactory[BaseExecutor]):
    pass


# --------------------------------------------------------------------------- flat runtime shared by none / ddp / fsdp
def _wants_flat(impl: str, model: nn.Module) -> bool:
    if impl == "torch":
        return False
    p = next(model.parameters(), None)
    on_cuda = p is not None and p.is_cuda
    if impl == "flat":
        return True
    return on_cuda  # "auto"


class FlatExecutor(BaseExecutor):
    """Single-process flat runtime; the distributed executors add the collectives."""

    flat_capable = True
    sharded = False

    def __init__(self, grad_accum_steps: int = 1, impl: str = "auto", overlap: bool = True):
        super().__init__(grad_accum_steps)
        if impl not in ("auto", "flat", "torch"):
            raise ValueError("impl must be 'auto', 'flat' or 'torch'")
        self.impl, self.overlap = impl, overlap
        self._comm_stream = None
        self._pending_units: List[FlatUnit] = []
        self.grad_scale: Optional[torch.Tensor] = None
        self.last_grad_norm: Optional[torch.Tensor] = None
        self._norm_done = False

    # -- set-up -------------------------------------------------------------------------------------------------
    def _prepare_model(self, model: nn.Module) -> nn.Module:
        if not _wants_flat(self.impl, model):
            return self._prepare_torch(model)
        self.engine = FlatParamEngine(model, get_world_size() if self.sharded else 1, get_rank() if self.sharded else 0,
                                      allocator=self._allocator(model))
        model._flat_engine = self.engine
        model._flat_executor = self
        self._init_comm(model)
        for unit in self.engine.units:
            for mname in unit.module_names:
                model.get_submodule(mname).register_forward_pre_hook(self._make_pre_hook(unit), with_kwargs=True)
        return model

    def _prepare_torch(self, model: nn.Module) -> nn.Module:
        return model

    def _allocator(self, model: nn.Module):
        return None

    def _init_comm(self, model: nn.Module):
        if self.use_distributed and next(model.parameters()).is_cuda:
            self._comm_stream = torch.cuda.Stream()

    # -- readiness tracking ---------------------------------------------------------------------------------------
    def _make_pre_hook(self, unit: FlatUnit):
        def hook(module, args, kwargs):
            self._before_unit_forward(unit)
            if not torch.is_grad_enabled():
                return None
            for a in list(args) + list(kwargs.values()):
                if isinstance(a, torch.Tensor) and a.requires_grad:
                    a.register_hook(lambda g, u=unit: self._unit_backward_done(u))
                    break
            return None

        return hook

    def _before_unit_forward(self, unit: FlatUnit):
        pass

    def before_param_use(self, p) -> None:
        unit = getattr(p, "_flat_unit", None)
        if unit is not None and self.engine is not None:
            self._before_unit_forward(unit)

    def _unit_backward_done(self, unit: FlatUnit):
        if unit.ready:
            return
        unit.ready = True
        if self.gradient_state.sync_gradients and self.overlap:
            self._reduce_unit(unit)

    def _reduce_unit(self, unit: FlatUnit):
        unit.reduced = True

    def backward(self, loss: torch.Tensor, gradient: Optional[torch.Tensor] = None):
        if self.engine is not None:
            for u in self.engine.units:
                u.ready = u.reduced = False
        loss.backward(gradient)
        if self.engine is not None and self.gradient_state.sync_gradients:
            for u in reversed(self.engine.units):
                u.ready = True
                if not u.reduced:
                    self._reduce_unit(u)
            self._finish_reductions()

    def _finish_reductions(self):
        if self._comm_stream is not None:
            torch.cuda.current_stream().wait_stream(self._comm_stream)

    # -- clipping: the coefficient stays on the device ------------------------------------------------------------------
    def _averaging_scale(self) -> float:
        return 1.0

    def clip_grad_norm(self, model: nn.Module, max_norm: float) -> float:
        if self.engine is None:
            return self._clip_torch(model, max_norm)
        from astrai_b200 import ops

        sumsq = self._grad_sumsq()
        if self.sharded and self.use_distributed:
            dist.all_reduce(sumsq)
        self._norm_done = True
        self.grad_scale, self.last_grad_norm = ops.clip_coef(sumsq, max_norm, self._averaging_scale())
        norm = float(self.last_grad_norm.item())
        self._after_norm_sync()
        return norm

    def _grad_sumsq(self) -> torch.Tensor:
        return self.engine.grad_sumsq(sharded=self.sharded)

    def _after_norm_sync(self):
        pass

    def _clip_torch(self, model, max_norm):
        return super().clip_grad_norm(model, max_norm)

    # -- optimizer-step plumbing ------------------------------------------------------------------------------------
    def _effective_scale(self) -> Optional[torch.Tensor]:
        if self.grad_scale is not None:
            return self.grad_scale
        s = self._averaging_scale()
        if s == 1.0:
            return None
        return torch.full((1,), s, dtype=torch.float32, device=self.engine.units[0].grad_buf.device)

    def _before_optimizer_step(self, optimizer):
        if self.engine is None:
            return
        self._ensure_step_barrier()
        if getattr(optimizer, "supports_flat", False):
            optimizer.bind_flat(self.engine, self._effective_scale(), sharded=self.sharded, fused=self._fused_runtime())
        else:
            if self.sharded:
                raise RuntimeError("the sharded flat runtime needs an optimizer with flat support (FusedAdamW)")
            self.engine.materialize_grads(self._effective_scale())

    def _ensure_step_barrier(self):
        pass

    def _fused_runtime(self):
        return None

    def _after_optimizer_step(self, optimizer):
        if self.engine is None:
            return
        self.grad_scale = None
        self._norm_done = False
        if not getattr(optimizer, "supports_flat", False):
            self.engine.drop_grads()
        self._after_flat_update()

    def _after_flat_update(self):
        pass

    def _zero_grad(self, optimizer) -> bool:
        if self.engine is None:
            return False
        if not (getattr(optimizer, "supports_flat", False) and getattr(optimizer, "zeroed_in_step", False)):
            self.engine.zero_grad()
        return True


@ExecutorFactory.register("none")
class NoneExecutor(FlatExecutor):
    """Single device.  On CUDA the flat runtime is used (fp32 main_grad, fused q/k/v and gate/up GEMMs)."""


@ExecutorFactory.register("ddp")
class DDPExecutor(FlatExecutor):
    """Data parallel: replicated parameters, gradients summed across ranks once per optimizer step.

    Flat runtime: one NCCL all-reduce per unit over its fp32 gradient buffer, issued on a side stream as soon as
    the unit's backward pass has finished on the last micro-batch; the ``1/world`` average is folded into the clip
    coefficient.  ``impl="torch"`` wraps ``DistributedDataParallel`` with the reference's constructor arguments
    (``astrai/parallel/executor.py:254-312``).
    """

    def __init__(self, grad_accum_steps: int = 1, impl: str = "auto", overlap: bool = True, dim: int = 0,
                 broadcast_buffers: bool = True, init_sync: bool = True, process_group=None, bucket_cap_mb: int = 25,
                 find_unused_parameters: bool = False, gradient_as_bucket_view: bool = False,
                 static_graph: bool = False, mixed_precision=None, device_mesh=None, check_reduction: bool = False,
                 delay_all_reduce_named_params=None, param_to_hook_all_reduce=None):
        super().__init__(grad_accum_steps, impl, overlap)
        # the last three only mean something to ``impl="torch"`` (they are DistributedDataParallel's own arguments)
        self._ddp_kwargs = dict(dim=dim, broadcast_buffers=broadcast_buffers, init_sync=init_sync,
                                process_group=process_group, bucket_cap_mb=bucket_cap_mb,
                                find_unused_parameters=find_unused_parameters,
                                gradient_as_bucket_view=gradient_as_bucket_view, static_graph=static_graph,
                                mixed_precision=mixed_precision, device_mesh=device_mesh, check_reduction=check_reduction,
                                delay_all_reduce_named_params=delay_all_reduce_named_params,
                                param_to_hook_all_reduce=param_to_hook_all_reduce)
        self._group = process_group

    def _prepare_model(self, model):
        model = super()._prepare_model(model)
        if self.engine is not None and self.use_distributed and self._ddp_kwargs["init_sync"]:
            for u in self.engine.units:
                dist.broadcast(u.param_buf, src=0, group=self._group)
        return model

    def _prepare_torch(self, model):
        from torch.nn.parallel import DistributedDataParallel as DDP

        if not self.use_distributed:
            logger.warning("DDP backend selected but world_size=1, model not wrapped")
            return model
        kw = {k: v for k, v in self._ddp_kwargs.items() if v is not None or k == "process_group"}
        if next(model.parameters()).is_cuda:
            local = int(os.environ.get("LOCAL_RANK", get_rank()))
            return DDP(model, device_ids=[local], output_device=local, **kw)
        return DDP(model, **kw)

    def _no_sync(self, model):
        from torch.nn.parallel import DistributedDataParallel as DDP

        return model.no_sync() if isinstance(model, DDP) else contextlib.nullcontext()

    def unwrap_model(self, model):
        from torch.nn.parallel import DistributedDataParallel as DDP

        return (model.module if isinstance(model, DDP) else model).state_dict()

    def _averaging_scale(self) -> float:
        return 1.0 / get_world_size() if self.use_distributed else 1.0

    def _reduce_unit(self, unit: FlatUnit):
        unit.reduced = True
        if not self.use_distributed:
            return
        if self._comm_stream is not None:
            self._comm_stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self._comm_stream):
                dist.all_reduce(unit.grad_buf, group=self._group)
        else:
            dist.all_reduce(unit.grad_buf, group=self._group)


@ExecutorFactory.register("fsdp")
class FSDPExecutor(FlatExecutor):
    """Fully sharded data parallel.

    Flat runtime: each rank owns shard ``r`` of every unit for the fp32 master weights and Adam moments.
    During an accumulation window gradients accumulate locally in the unit's fp32 buffer (the reference does the
    same through ``set_requires_gradient_sync(False)``, ``astrai/parallel/executor.py:363-375``); on the closing
    micro-batch each unit is reduce-scattered as soon as its backward pass is done, overlapped with the remaining
    backward work.  After the sharded update every unit's parameters are all-gathered on the side stream and the
    next forward pass waits per unit, so the gather of unit ``i+1`` overlaps the compute of unit ``i``.  With
    ``comm="p2p"`` the reduce-scatter, the AdamW update and the all-gather of a unit run as fused kernels over
    NVLink peer memory (:mod:`astrai_b200.parallel.fused_fsdp`).  ``impl="torch"`` applies FSDP2 ``fully_shard``
    to each direct child exactly as the reference does (``executor.py:338-361``).

    ``reshard=True`` (flat runtime, library collectives) is the full-shard placement: parameters and gradients are whole
    only while their unit computes, every micro-batch gathers and reduce-scatters
    (:mod:`astrai_b200.parallel.fsdp_reshard`).  The default keeps bf16 parameters and the fp32 gradient buffer whole
    on every rank and shards the optimizer state and master weights; it communicates once per optimizer step.
    """

    sharded = True

    def __init__(self, grad_accum_steps: int = 1, impl: str = "auto", overlap: bool = True, comm: str = "nccl",
                 comm_timeout_s: float = 120.0, mesh: Optional[Any] = None, mp_policy: Optional[Any] = None,
                 reshard_after_forward: bool = False, reshard: bool = False):
        super().__init__(grad_accum_steps, impl, overlap)
        if comm not in ("nccl", "p2p", "nvls"):
            raise ValueError("comm must be 'nccl', 'p2p' or 'nvls'")
        if reshard and comm != "nccl":
            raise ValueError("reshard=True releases and re-creates the unit buffers, which symmetric memory cannot do: use comm='nccl'")
        self.reshard = bool(reshard)
        self._rs: Optional[Any] = None
        self.communicates_every_micro_batch = self.reshard
        self.comm = comm
        self.comm_timeout_s = float(comm_timeout_s)
        self._mesh, self._mp_policy, self._reshard_after_forward = mesh, mp_policy, reshard_after_forward
        self._gather_events: Dict[str, Any] = {}
        self._fused = None

    # -- torch FSDP2 path ------------------------------------------------------------------------------------------
    def _prepare_torch(self, model):
        if not self.use_distributed:
            logger.warning("FSDP backend selected but world_size=1, model not wrapped")
            return model
        from torch.distributed.fsdp import fully_shard

        kw = {k: v for k, v in dict(mesh=self._mesh, mp_policy=self._mp_policy,
                                    reshard_after_forward=self._reshard_after_forward).items() if v is not None}
        for child in model.children():
            for sub in (child if isinstance(child, nn.ModuleList) else [child]):
                fully_shard(sub, **kw)
        return model

    @contextmanager
    def _no_sync(self, model):
        if self.engine is not None:
            yield
            return
        from torch.distributed.fsdp import FSDPModule

        mods = [m for m in model.modules() if isinstance(m, FSDPModule)]
        for m in mods:
            m.set_requires_gradient_sync(False, recurse=True)
        try:
            yield
        finally:
            for m in mods:
                m.set_requires_gradient_sync(True, recurse=True)

    def _clip_torch(self, model, max_norm):
        if not self.use_distributed:
            return BaseExecutor.clip_grad_norm(self, model, max_norm)
        from torch.distributed.tensor import DTensor

        grads = [p.grad for p in model.parameters() if p.grad is not None]
        local = torch.nn.utils.get_total_norm(grads)
        if isinstance(local, DTensor):
            local = local.to_local()
        sq = local.float() ** 2
        dist.all_reduce(sq)
        total = sq.sqrt()
        coef = torch.clamp(max_norm / (total + 1e-6), max=1.0)
        for g in grads:
            g.mul_(coef)
        return total.item()

    def local_state_dict(self, model):
        if (self.engine is None or self._rs is not None) and self.use_distributed:
            return None  # FSDP2 DTensor shards / parameters released at rest: the full weights need the peers
        return model.state_dict()  # flat runtime: bf16 parameters are replicated; pending gathers are not waited for

    def unwrap_model(self, model):
        if self._rs is not None:
            self._rs.unshard_all()  # collective: every rank passes through here (checkpoint_context)
            sd = {k: v.clone() for k, v in model.state_dict().items()} if (get_rank() == 0 or not self.use_distributed) else None
            self._rs.release_all()
            return sd
        if self.engine is not None or not self.use_distributed:
            self._wait_all_gathers()
            return model.state_dict() if (get_rank() == 0 or not self.use_distributed) else None
        from torch.distributed.fsdp import FSDPModule
        from torch.distributed.tensor import DTensor

        mods = [m for m in model.modules() if isinstance(m, FSDPModule)]
        for m in mods:
            m.unshard()
        out = {}
        for k, v in model.state_dict().items():
            full = v.full_tensor() if isinstance(v, DTensor) else v
            if get_rank() == 0:
                out[k] = full
        for m in mods:
            m.reshard()
        return out if get_rank() == 0 else None

    # -- flat path --------------------------------------------------------------------------------------------------
    def _allocator(self, model: nn.Module):
        if self.comm == "nccl" or not self.use_distributed:
            return None
        from astrai_b200.parallel.fused_fsdp import SymmetricAllocator, arena_bytes_for
        from astrai_b200.parallel.symm import SymmetricArena

        dev = next(model.parameters()).device
        try:
            arena = SymmetricArena(arena_bytes_for(model, get_world_size()), dev)
        except Exception as exc:  # noqa: BLE001 - no peer mapping on this machine (every rank fails alike)
            logger.warning("symmetric memory unavailable (%s); FSDP falls back to NCCL collectives", exc)
            self.comm = "nccl"
            return None
        if self.comm == "nvls" and not arena.has_multicast:
            logger.warning("no NVSwitch multicast mapping; using plain peer loads / stores")
            self.comm = "p2p"
        self._symm = SymmetricAllocator(arena)
        return self._symm.alloc

    def _init_comm(self, model):
        super()._init_comm(model)
        eng = self.engine
        dev = eng.units[0].param_buf.device
        for u in eng.units:
            u.grad_shard = torch.zeros(u.shard_size, dtype=torch.float32, device=dev)
        if self.use_distributed:
            for u in eng.units:  # rank 0's initial weights everywhere
                dist.broadcast(u.param_buf, src=0)
        if self.reshard:
            from astrai_b200.parallel.fsdp_reshard import ReshardRuntime

            self._rs = ReshardRuntime(eng, self._comm_stream, reshard_after_forward=True)
            for u in eng.units:
                for mname in u.module_names:
                    model.get_submodule(mname).register_forward_hook(lambda mod, args, out, u=u: self._rs.after_forward(u, out))
            return
        if self.use_distributed:
            if self.comm != "nccl":
                from astrai_b200.parallel.fused_fsdp import FusedFSDP

                self._fused = FusedFSDP(eng, self._symm, mode=self.comm, timeout_s=self.comm_timeout_s)
                self._symm.arena.barrier()  # every rank's buffers hold the broadcast weights before anyone proceeds

    def _averaging_scale(self) -> float:
        return 1.0 / get_world_size() if self.use_distributed else 1.0

    def _unit_backward_done(self, unit: FlatUnit):
        if self._rs is None:
            return super()._unit_backward_done(unit)
        if not unit.ready:  # every micro-batch: the full gradient buffer does not outlive the unit's backward pass
            unit.ready = True
            self._reduce_unit(unit)

    def backward(self, loss: torch.Tensor, gradient: Optional[torch.Tensor] = None):
        if self._rs is None:
            return super().backward(loss, gradient)
        for u in self.engine.units:
            u.ready = u.reduced = False
        self._rs.begin_backward()
        loss.backward(gradient)
        for u in reversed(self.engine.units):  # what no hook saw finish (the embedding's unit), and unused units
            u.ready = True
            if not u.reduced:
                self._reduce_unit(u)
        self._rs.finish()

    def _reduce_unit(self, unit: FlatUnit):
        unit.reduced = True
        if self._rs is not None:
            self._rs.reduce(unit)
            return
        if not self.use_distributed:
            unit.grad_shard = unit.grad_buf[: unit.shard_size]
            return
        if self._fused is not None:
            self._fused.reduce_scatter(unit, self._comm_stream)
            return
        if self._comm_stream is not None:
            self._comm_stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self._comm_stream):
                dist.reduce_scatter_tensor(unit.grad_shard, unit.grad_buf)
        else:
            dist.reduce_scatter_tensor(unit.grad_shard, unit.grad_buf)

    def _after_flat_update(self):
        """Parameters of every unit were updated in the owner's shard only: gather them, overlapped with what follows."""
        if self._rs is not None:
            self._rs.release_all()  # whatever is still whole holds the old values; the next forward pass gathers
            return
        if not self.use_distributed:
            return
        if self._fused is not None and self._fused.gathers_in_update:
            return
        stream = self._comm_stream
        if stream is not None:
            stream.wait_stream(torch.cuda.current_stream())
        for u in self.engine.units:
            ctx = torch.cuda.stream(stream) if stream is not None else contextlib.nullcontext()
            with ctx:
                dist.all_gather_into_tensor(u.param_buf, u.param_shard(self.engine.rank))
                if stream is not None:
                    ev = torch.cuda.Event()
                    ev.record(stream)
                    self._gather_events[u.name] = ev

    def _fused_runtime(self):
        return self._fused

    def _grad_sumsq(self) -> torch.Tensor:
        if self._fused is not None:
            return self._fused.take_sumsq()
        return super()._grad_sumsq()

    def _after_norm_sync(self):
        if self._fused is not None:
            self._fused.check()

    def _ensure_step_barrier(self):
        """The fused kernels write into peers' parameter buffers: every rank must have finished its backward pass and
        its reads of the peers' gradients first.  The norm all-reduce is that barrier; run it if nobody clipped."""
        if self._fused is not None and not self._norm_done:
            self.clip_grad_norm(None, None)

    def _before_unit_forward(self, unit: FlatUnit):
        if self._rs is not None:
            self._rs.before_forward(unit)
            return
        if self._fused is not None:
            self._fused.wait_params(unit)
        ev = self._gather_events.pop(unit.name, None)
        if ev is not None:
            torch.cuda.current_stream().wait_event(ev)

    def _wait_all_gathers(self):
        if self._fused is not None:
            self._fused.wait_all_params()
        for ev in self._gather_events.values():
            torch.cuda.current_stream().wait_event(ev)
        self._gather_events.clear()

    def _zero_grad(self, optimizer) -> bool:
        if self.engine is None:
            return False
        if self._rs is not None:
            self._rs.zero_accumulators()  # the full buffers are created zeroed for each backward pass
            return True
        self.engine.zero_grad()  # the full buffers; the update consumed the reduced shards
        return True
