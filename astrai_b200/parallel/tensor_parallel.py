"""Tensor parallelism with sequence-sharded activations, fused with its collectives over NVLink peer memory.

Megatron-style pairing inside one NVSwitch domain (``tp_size`` <= 8):

* :class:`ColumnParallelLinear` (q/k/v, gate/up): every rank holds ``N/tp`` output columns of the weight and a
  ``[tokens/tp, K]`` slice of the input.  Forward is ``all-gather -> GEMM`` in ONE kernel (``tp_gemm_allgather_``):
  copy CTAs pull the peers' slices into the local symmetric buffer while the tcgen05 CTAs already multiply the
  slices that arrived.  Backward: ``dX = reduce-scatter(dY W)`` in one kernel, ``dW = dY^T X_full`` locally.
* :class:`RowParallelLinear` (o_proj, down): every rank holds ``K/tp`` input columns; forward is ``GEMM ->
  reduce-scatter`` in ONE kernel (``tp_gemm_reducescatter_``): tiles are stored straight into the owner rank's staging
  slot and the owner sums them in a fixed order.  Backward: ``dX = all-gather(dY) W`` fused the same way.

``comm="nccl"`` runs the same math as ``all_gather_into_tensor`` / ``reduce_scatter_tensor`` around the plain tcgen05
GEMM; it is the comparison baseline and the path taken on CPU (Gloo) tests.

The reference accepts ``--tp_size`` and drops it (``scripts/tools/train.py:513-519``); there is no counterpart.
Buffers are double-buffered by call parity: a rank can run at most one fused call ahead of its slowest peer (each call
needs every peer's flag of the same epoch), so a buffer of parity ``p`` is never rewritten while a peer still reads it.
"""

from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn
from torch import Tensor
from torch.autograd import Function

from astrai_b200.parallel import symm

TILE_ROWS = 128


class TPContext:
    """Per-process state of the fused tensor-parallel kernels: arena, flag array, epochs and buffer pools."""

    MAX_UNITS = 64

    def __init__(self, arena, rank: int, world: int, timeout_s: float = 60.0, n_copy_ctas: int = 16,
                 fuse_reduce: bool = True, group=None, engine: str = "pair"):
        """``engine="pair"``: the CTA-pair kernels with in-kernel bulk-copy transfer (``ops/csrc/gemm_comm2.cu``) whenever
        a row block is a whole number of 256-row pair tiles, else (and with ``engine="single"``) the one-CTA-per-tile
        kernels with copy CTAs and epilogue peer stores (``gemm_comm.cu``)."""
        self.engine = engine
        self.copy_slots = 0  # pair engine: shared-memory copy slots of the comm lane; 0 = chosen from the shape per call
        self.arena, self.rank, self.world = arena, rank, world
        self.timeout_s, self.n_copy_ctas, self.fuse_reduce = float(timeout_s), int(n_copy_ctas), bool(fuse_reduce)
        self.group = group
        self.flags = arena.alloc_flags(self.MAX_UNITS)
        self._gather: Dict[Tuple[int, int, int], symm.SymmBuffer] = {}
        self._stage: Dict[Tuple[int, int, int], symm.SymmBuffer] = {}
        self._epoch = {"ag": 0, "rs": 0}
        dev = self.flags.tensor.device
        self.chunk_flags = torch.zeros(8, dtype=torch.int32, device=dev)
        self.chunk_counter = torch.zeros(8, dtype=torch.int32, device=dev)
        self.tile_counter = torch.zeros(8, dtype=torch.int32, device=dev)
        self.pull_counter = torch.zeros(1, dtype=torch.int32, device=dev)
        self._gathered: Dict[Tuple[int, int], Tensor] = {}

    # The pools are keyed by shape and parity; allocation order must be identical on every rank (it is: the same
    # model code runs everywhere), because a sub-buffer is identified by its offset in the arena.
    def gather_buffer(self, m: int, k: int, parity: int) -> symm.SymmBuffer:
        key = (m, k, parity)
        if key not in self._gather:
            self._gather[key] = self.arena.alloc(m * k, torch.bfloat16, zero=False)
        return self._gather[key]

    def own_rows_buffer(self, ms: int, k: int, parity: int) -> symm.SymmBuffer:
        """This rank's ``[ms, k]`` rows of an all-gather, where the peers' copy warps read them."""
        key = ("own", ms, k, parity)
        if key not in self._gather:
            self._gather[key] = self.arena.alloc(ms * k, torch.bfloat16, zero=False)
        return self._gather[key]

    def stage_buffer(self, rows: int, n: int, parity: int) -> symm.SymmBuffer:
        key = (rows, n, parity)
        if key not in self._stage:
            self._stage[key] = self.arena.alloc(self.world * rows * n, torch.bfloat16, zero=False)
        return self._stage[key]

    def gathered_buffer(self, rows: int, n: int) -> Tensor:
        """Local (not peer-visible) landing area of the pulled partial blocks: ``[world, rows, n]`` bf16."""
        key = (rows, n)
        if key not in self._gathered:
            self._gathered[key] = torch.empty(self.world * rows * n, dtype=torch.bfloat16, device=self.flags.tensor.device)
        return self._gathered[key]

    def pair_engine(self, m: int) -> bool:
        return self.engine == "pair" and m % (self.world * 256) == 0

    def next_epoch(self, kind: str) -> int:
        self._epoch[kind] += 1
        return self._epoch[kind]


_CTX: Optional[TPContext] = None
_GROUP = {"group": None, "rank": 0, "world": None}  # the tensor-parallel process group when it is not WORLD


def set_context(ctx: Optional[TPContext]):
    global _CTX
    _CTX = ctx


def set_group(group, rank: int, world: int):
    """Name the tensor-parallel group for the collective (``comm="nccl"``) path; ``world=None`` means WORLD."""
    _GROUP.update(group=group, rank=rank, world=world)


def _group_world(ctx: Optional["TPContext"]):
    if ctx is not None:
        return ctx.group, ctx.world
    if _GROUP["world"] is not None:
        return _GROUP["group"], _GROUP["world"]
    return None, (dist.get_world_size() if dist.is_initialized() else 1)


def get_context() -> Optional[TPContext]:
    return _CTX


def init_tensor_parallel(arena_bytes: int = 1 << 30, timeout_s: float = 60.0, group=None) -> TPContext:
    """Collective: create the symmetric arena of the tensor-parallel group and install the context."""
    arena = symm.SymmetricArena(arena_bytes, group=group)
    ctx = TPContext(arena, arena.rank, arena.world_size, timeout_s=timeout_s, group=group)
    set_context(ctx)
    return ctx


# --------------------------------------------------------------------------- the two fused primitives
def _fusable(rows_total: int, world: int, *tensors: Tensor) -> bool:
    return (all(t.is_cuda and t.dtype == torch.bfloat16 for t in tensors) and rows_total % (world * TILE_ROWS) == 0)


def allgather_gemm(x_local: Tensor, w: Tensor, w_kmajor: bool = True, ctx: Optional[TPContext] = None,
                   comm: str = "p2p") -> Tuple[Tensor, Tensor]:
    """``(concat_r x_r) @ op(w)``; returns ``(y [M, N], x_full [M, K])`` (``x_full`` is kept for the weight gradient).

    ``w`` is ``[N, K]`` (``w_kmajor``) or ``[K, N]``."""
    ctx = ctx or _CTX
    group, world = _group_world(ctx)
    ms, k = x_local.shape
    m = ms * world
    n = w.shape[0] if w_kmajor else w.shape[1]
    if comm == "p2p" and ctx is not None and _fusable(m, world, x_local, w) and n % 32 == 0 and k % 8 == 0:
        epoch = ctx.next_epoch("ag")
        y = torch.empty((m, n), dtype=torch.bfloat16, device=x_local.device)
        if ctx.pair_engine(m):
            # Only this rank's own rows live in symmetric memory (where the peers read them); the gathered matrix is
            # a plain tensor of this call, so autograd can keep it for the weight gradient without a copy.  The kernel
            # reads rank r's rows at `ptr[r] + r * block` and writes them at `ptr[rank] + r * block`: the peers'
            # pointers are therefore biased back by their block offset and this rank's pointer is the new tensor.
            own = ctx.own_rows_buffer(ms, k, epoch & 1)
            own.tensor.view(ms, k).copy_(x_local)
            x_full = torch.empty((m, k), dtype=torch.bfloat16, device=x_local.device)
            x_full[ctx.rank * ms:(ctx.rank + 1) * ms].copy_(x_local)
            blk = ms * k * 2
            ptrs = [x_full.data_ptr() if r == ctx.rank else own.peer_ptrs[r] - r * blk for r in range(world)]
            torch.ops.astrai_b200.tp2_gemm_allgather_(ptrs, w.contiguous(), w_kmajor, y, ctx.flags.peer_ptrs,
                                                      ctx.chunk_flags, ctx.chunk_counter, ctx.rank, 0, ctx.MAX_UNITS, epoch,
                                                      ctx.timeout_s, ctx.copy_slots)
            return y, x_full
        buf = ctx.gather_buffer(m, k, epoch & 1)
        x_full = buf.tensor.view(m, k)
        x_full[ctx.rank * ms:(ctx.rank + 1) * ms].copy_(x_local)
        torch.ops.astrai_b200.tp_gemm_allgather_(buf.peer_ptrs, w.contiguous(), w_kmajor, y, ctx.flags.peer_ptrs,
                                                 ctx.chunk_flags, ctx.chunk_counter, ctx.rank, 0, ctx.MAX_UNITS, epoch,
                                                 ctx.timeout_s, ctx.n_copy_ctas)
        return y, x_full.clone()  # the symmetric buffer is reused two calls later: hand out a copy
    if world > 1:
        x_full = torch.empty((m, k), dtype=x_local.dtype, device=x_local.device)
        dist.all_gather_into_tensor(x_full, x_local.contiguous(), group=group)
    else:
        x_full = x_local
    from astrai_b200 import ops

    y = ops.gemm(x_full, w, b_kmajor=w_kmajor) if x_full.is_cuda else (x_full @ (w.t() if w_kmajor else w))
    return y, x_full


def gemm_reducescatter(x: Tensor, w: Tensor, w_kmajor: bool = True, ctx: Optional[TPContext] = None,
                       comm: str = "p2p") -> Tensor:
    """Row block ``rank`` of ``sum_p x_p @ op(w_p)``: ``x [M, K_p]`` -> ``[M / world, N]``."""
    ctx = ctx or _CTX
    group, world = _group_world(ctx)
    m, k = x.shape
    n = w.shape[0] if w_kmajor else w.shape[1]
    ms = m // world
    if comm == "p2p" and ctx is not None and _fusable(m, world, x, w) and n % 32 == 0 and k % 8 == 0:
        epoch = ctx.next_epoch("rs")
        st = ctx.stage_buffer(ms, n, epoch & 1)
        out = torch.empty((ms, n), dtype=torch.bfloat16, device=x.device)
        if ctx.pair_engine(m) and ctx.fuse_reduce:
            # the staging area doubles as this rank's whole partial product [M, N]; the peers' blocks are pulled from it
            torch.ops.astrai_b200.tp2_gemm_reducescatter_(x.contiguous(), w.contiguous(), w_kmajor, st.peer_ptrs,
                                                          ctx.gathered_buffer(ms, n), out, ctx.flags.peer_ptrs, ctx.tile_counter,
                                                          ctx.pull_counter, ctx.rank, 1, ctx.MAX_UNITS, epoch, ctx.timeout_s, 1,
                                                          ctx.copy_slots)
            return out
        torch.ops.astrai_b200.tp_gemm_reducescatter_(x.contiguous(), w.contiguous(), w_kmajor, st.peer_ptrs, out,
                                                     ctx.flags.peer_ptrs, ctx.tile_counter, ctx.rank, 1, ctx.MAX_UNITS, epoch,
                                                     ctx.timeout_s, ctx.fuse_reduce)
        if not ctx.fuse_reduce:
            ctx._pending_reduce = (st, out)  # the caller reduces after every emulated rank has scattered
        return out
    from astrai_b200 import ops

    full = ops.gemm(x, w, b_kmajor=w_kmajor) if x.is_cuda else (x @ (w.t() if w_kmajor else w))
    if world == 1:
        return full
    out = torch.empty((ms, n), dtype=full.dtype, device=full.device)
    dist.reduce_scatter_tensor(out, full.contiguous(), group=group)
    return out


# --------------------------------------------------------------------------- autograd + modules
class _GatherRowValues(Function):
    """Per-row scalars of this rank's token rows -> the values of every row of the block, on every rank.

    For objectives that are not sums over tokens (sequence log-probabilities of preference and policy-gradient losses):
    every rank then computes the SAME loss from the same full vector.  The executors average gradients over the ranks
    of a block (their convention is one partial loss per rank), so the backward hands this rank's slice of the incoming
    gradient back multiplied by the block size: summed over the block and divided by its size, that is the gradient of
    the loss counted once."""

    @staticmethod
    def forward(ctx, values, group, rank, world):
        ctx.rank, ctx.world, ctx.n = rank, world, values.numel()
        full = torch.empty(world * values.numel(), dtype=values.dtype, device=values.device)
        dist.all_gather_into_tensor(full, values.contiguous(), group=group)
        return full

    @staticmethod
    def backward(ctx, g):
        return g[ctx.rank * ctx.n:(ctx.rank + 1) * ctx.n] * float(ctx.world), None, None, None


def gather_row_values(values: Tensor) -> Tensor:
    """``[rows / tp]`` values of the local token rows -> ``[rows]`` on every rank of the tensor-parallel group
    (differentiable; see :class:`_GatherRowValues`)."""
    group, world = _group_world(get_context())
    if world <= 1:
        return values
    return _GatherRowValues.apply(values, group, dist.get_rank(group), world)


class _ColumnParallelFn(Function):
    @staticmethod
    def forward(ctx, x_local, w, comm):
        y, x_full = allgather_gemm(x_local, w, True, comm=comm)
        ctx.save_for_backward(x_full, w)
        ctx.comm = comm
        return y

    @staticmethod
    def backward(ctx, gy):
        from astrai_b200 import ops

        x_full, w = ctx.saved_tensors
        gy = gy.contiguous()
        dx = gemm_reducescatter(gy, w, False, comm=ctx.comm)  # dY [M, N_r] @ W_r [N_r, K], summed over ranks, row block
        mg = getattr(w, "main_grad", None)
        if mg is not None:  # the flat runtime's fp32 gradient buffer: accumulate in place (wgrad epilogue on CUDA)
            if gy.is_cuda:
                ops.gemm(gy, x_full, out=mg, a_kmajor=False, b_kmajor=False, out_f32=True, accumulate=True)
            else:
                mg.add_(gy.float().t() @ x_full.float())
            return dx, None, None
        dw = ops.gemm(gy, x_full, a_kmajor=False, b_kmajor=False) if gy.is_cuda else gy.t() @ x_full
        return dx, dw, None


class _RowParallelFn(Function):
    @staticmethod
    def forward(ctx, x, w, comm):
        ctx.save_for_backward(x, w)
        ctx.comm = comm
        return gemm_reducescatter(x, w, True, comm=comm)

    @staticmethod
    def backward(ctx, gy_local):
        from astrai_b200 import ops

        x, w = ctx.saved_tensors
        dx, gy_full = allgather_gemm(gy_local.contiguous(), w, False, comm=ctx.comm)  # AG(dY) [M, N] @ W_p [N, K_p]
        mg = getattr(w, "main_grad", None)
        if mg is not None:
            if x.is_cuda:
                ops.gemm(gy_full, x, out=mg, a_kmajor=False, b_kmajor=False, out_f32=True, accumulate=True)
            else:
                mg.add_(gy_full.float().t() @ x.float())
            return dx, None, None
        dw = ops.gemm(gy_full, x, a_kmajor=False, b_kmajor=False) if x.is_cuda else gy_full.t() @ x
        return dx, dw, None


class ColumnParallelLinear(nn.Module):
    """``[tokens/tp, in] -> [tokens, out/tp]``; this rank's weight is rows ``[rank*out/tp, (rank+1)*out/tp)``."""

    def __init__(self, in_features: int, out_features: int, tp_size: int, tp_rank: int, init_std: float = 0.02,
                 comm: str = "p2p", dtype=None, device=None):
        super().__init__()
        if out_features % tp_size:
            raise ValueError("out_features must be divisible by tp_size")
        self.tp_size, self.tp_rank, self.comm = tp_size, tp_rank, comm
        self.weight = nn.Parameter(torch.empty(out_features // tp_size, in_features, dtype=dtype, device=device))
        nn.init.normal_(self.weight, std=init_std)

    def forward(self, x_local: Tensor) -> Tensor:
        return _ColumnParallelFn.apply(x_local.reshape(-1, x_local.shape[-1]), self.weight, self.comm)

    @staticmethod
    def shard(full_weight: Tensor, tp_size: int, tp_rank: int) -> Tensor:
        rows = full_weight.shape[0] // tp_size
        return full_weight[tp_rank * rows:(tp_rank + 1) * rows].contiguous()


class RowParallelLinear(nn.Module):
    """``[tokens, in/tp] -> [tokens/tp, out]``; this rank's weight is columns ``[rank*in/tp, (rank+1)*in/tp)``."""

    def __init__(self, in_features: int, out_features: int, tp_size: int, tp_rank: int, init_std: float = 0.02,
                 comm: str = "p2p", dtype=None, device=None):
        super().__init__()
        if in_features % tp_size:
            raise ValueError("in_features must be divisible by tp_size")
        self.tp_size, self.tp_rank, self.comm = tp_size, tp_rank, comm
        self.weight = nn.Parameter(torch.empty(out_features, in_features // tp_size, dtype=dtype, device=device))
        nn.init.normal_(self.weight, std=init_std)

    def forward(self, x: Tensor) -> Tensor:
        return _RowParallelFn.apply(x.reshape(-1, x.shape[-1]), self.weight, self.comm)

    @staticmethod
    def shard(full_weight: Tensor, tp_size: int, tp_rank: int) -> Tensor:
        cols = full_weight.shape[1] // tp_size
        return full_weight[:, tp_rank * cols:(tp_rank + 1) * cols].contiguous()


class TensorParallelMLP(nn.Module):
    """SwiGLU feed-forward with sequence-sharded input and output: column-parallel gate/up (one fused all-gather ->
    GEMM over the stacked weight), SwiGLU on the local columns, row-parallel down (GEMM -> reduce-scatter)."""

    def __init__(self, dim: int, hidden: int, tp_size: int, tp_rank: int, comm: str = "p2p", dtype=None, device=None):
        super().__init__()
        self.hidden_local = hidden // tp_size
        self.gate_up = ColumnParallelLinear(dim, 2 * hidden, tp_size, tp_rank, comm=comm, dtype=dtype, device=device)
        self.down = RowParallelLinear(hidden, dim, tp_size, tp_rank, comm=comm, dtype=dtype, device=device)

    def forward(self, x_local: Tensor) -> Tensor:
        from astrai_b200 import ops

        gu = self.gate_up(x_local)  # [tokens, 2 * hidden / tp]: this rank's gate columns then its up columns
        return self.down(ops.swiglu_fused(gu))

    @staticmethod
    def shard_gate_up(gate: Tensor, up: Tensor, tp_size: int, tp_rank: int) -> Tensor:
        rows = gate.shape[0] // tp_size
        sl = slice(tp_rank * rows, (tp_rank + 1) * rows)
        return torch.cat([gate[sl], up[sl]], dim=0).contiguous()
