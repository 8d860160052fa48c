"""Context (sequence) parallel causal attention: the sequence is sharded over the ranks, K / V travel over NVLink.

Sharding is zig-zag: a sequence of ``S = 2 * W * c`` tokens is cut into ``2W`` chunks and rank ``r`` owns chunks ``r``
and ``2W - 1 - r`` - under a causal mask every rank then has the same amount of attention work.  Everything that is
per-token (projections, norms, MLP, loss) runs on the local ``2c`` tokens unchanged; only attention needs the others.

``comm="p2p"`` (the product): ONE attention launch also gathers K / V.  A few CTAs at the front of the grid pull the
peers' chunks from their symmetric memory (bulk copies, ring order) into a local gathered buffer and publish a flag
per source rank; the attention CTAs start on the chunks that are local and poll a chunk's flag before its first TMA
load (``ops/csrc/flash_fwd.cu``).  In the backward pass the dK / dV epilogue stores each key tile straight into the
staging slot of the rank that owns those keys and the owner sums the slots (``ops/csrc/flash_bwd.cu``): a
reduce-scatter without a collective call.  ``comm="nccl"`` is the baseline it is measured against: all-gather, the
same kernels on gathered tensors, reduce-scatter.

Model integration: after :func:`init_context_parallel` every causal dense attention call of the model
(``ops/attention.py::dense_attention``) is this op; the caller shards ``input_ids`` / ``target_ids`` with
:func:`zigzag_split` and passes ``position_ids = zigzag_positions(...)`` so that rotary embeddings see global positions.
Parameters are replicated over the context-parallel ranks, so their gradients are reduced like data-parallel ones.

The reference trains with data parallelism only (``astrai/parallel/setup.py:44-90``) and has no counterpart; sequence
length there is bounded by one GPU's activation memory.
"""

from __future__ import annotations

import math
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist
from torch import Tensor

from astrai_b200.parallel import symm

TILE = 128


# --------------------------------------------------------------------------- zig-zag layout helpers (any device)
def zigzag_split(x: Tensor, world: int, rank: int, dim: int = 1) -> Tensor:
    """The rows of ``x`` (full sequence along ``dim``) that rank ``rank`` owns: chunks ``rank`` and ``2W-1-rank``."""
    if x.size(dim) % (2 * world):
        raise ValueError(f"sequence length {x.size(dim)} is not a multiple of 2 * world = {2 * world}")
    chunks = x.chunk(2 * world, dim=dim)
    return torch.cat([chunks[rank], chunks[2 * world - 1 - rank]], dim=dim)


def zigzag_merge(parts: List[Tensor], dim: int = 1) -> Tensor:
    """Inverse of :func:`zigzag_split` given every rank's rows in rank order."""
    world = len(parts)
    chunks: List[Optional[Tensor]] = [None] * (2 * world)
    for r, p in enumerate(parts):
        a, b = p.chunk(2, dim=dim)
        chunks[r], chunks[2 * world - 1 - r] = a, b
    return torch.cat(chunks, dim=dim)


def zigzag_positions(seq_len: int, world: int, rank: int, device=None) -> Tensor:
    """Global positions of the local tokens (what rotary embeddings must be evaluated at)."""
    c = seq_len // (2 * world)
    return torch.cat([torch.arange(rank * c, (rank + 1) * c, device=device),
                      torch.arange((2 * world - 1 - rank) * c, (2 * world - rank) * c, device=device)])


# --------------------------------------------------------------------------- context
class CPContext:
    """Per-process state of context-parallel attention: arena, flags, epochs, double-buffered K/V source and staging."""

    def __init__(self, arena, rank: int, world: int, timeout_s: float = 60.0, n_copy_ctas: int = 8, group=None,
                 comm: str = "p2p"):
        if not 2 <= world <= symm.MAX_RANKS:
            raise ValueError(f"context parallel world size must be in 2..{symm.MAX_RANKS}")
        self.arena, self.rank, self.world, self.group, self.comm = arena, rank, world, group, comm
        self.timeout_s, self.n_copy_ctas = float(timeout_s), int(n_copy_ctas)
        self.active = True
        self._src: Dict[Tuple[int, int, int, int], symm.SymmBuffer] = {}
        self._stage: Dict[Tuple[int, int, int, int], symm.SymmBuffer] = {}
        self._epoch = {"fwd": 0, "bwd": 0}
        if arena is None:  # no peer memory (CPU ranks): only the collective statement of the op is available
            self.comm = "nccl"
            return
        self.flags = arena.alloc_flags(1)
        dev = self.flags.tensor.device
        self.chunk_state = torch.zeros(16, dtype=torch.int32, device=dev)   # landed flags | copy counters
        self.tile_counter = torch.zeros(8, dtype=torch.int32, device=dev)

    def paused(self):
        """Context manager: attention calls inside see no context parallelism (a model that runs on whole, unsharded
        sequences next to the sharded one, e.g. a generation pass)."""
        import contextlib

        @contextlib.contextmanager
        def cm():
            prev, self.active = self.active, False
            try:
                yield
            finally:
                self.active = prev

        return cm()

    # Buffers are keyed by shape and call parity.  Parity double-buffering is enough: a rank's launch n+1 cannot
    # finish before every peer's launch n+1 has started (it waits for their flags), i.e. before their launch n - the
    # last reader of the buffers of call n - has ended.  Allocation order is the same on every rank.
    def kv_source(self, batch: int, chunk: int, row: int, parity: int) -> symm.SymmBuffer:
        key = (batch, chunk, row, parity)
        if key not in self._src:
            self._src[key] = self.arena.alloc(2 * batch * 2 * chunk * row, torch.bfloat16, zero=False)
        return self._src[key]

    def stage(self, batch: int, chunk: int, row: int, parity: int) -> symm.SymmBuffer:
        key = (batch, chunk, row, parity)
        if key not in self._stage:
            self._stage[key] = self.arena.alloc(self.world * 2 * batch * 2 * chunk * row, torch.bfloat16, zero=False)
        return self._stage[key]

    def next_epoch(self, kind: str) -> int:
        self._epoch[kind] += 1
        return self._epoch[kind]


_CTX: Optional[CPContext] = None


def set_context(ctx: Optional[CPContext]):
    global _CTX
    _CTX = ctx


def get_context() -> Optional[CPContext]:
    return _CTX


def arena_bytes_for(batch: int, seq_len: int, world: int, n_kv_heads: int, head_dim: int) -> int:
    """Symmetric memory one attention shape needs: two K/V sources and two staging buffers plus flags and slack."""
    local = 2 * batch * (seq_len // world) * n_kv_heads * head_dim * 2  # K and V of the local rows, bf16
    return 2 * local + 2 * world * local + (1 << 20)


def init_context_parallel(arena_bytes: int, timeout_s: float = 60.0, group=None, n_copy_ctas: int = 8) -> CPContext:
    """Collective: create the symmetric arena of the context-parallel group and install the context."""
    arena = symm.SymmetricArena(arena_bytes, group=group)
    ctx = CPContext(arena, arena.rank, arena.world_size, timeout_s=timeout_s, n_copy_ctas=n_copy_ctas, group=group)
    set_context(ctx)
    return ctx


def init_context_parallel_group(group=None) -> CPContext:
    """Context without peer memory (CPU / Gloo ranks, or a baseline run): attention gathers keys with collectives."""
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    ctx = CPContext(None, rank, world, group=group, comm="nccl")
    set_context(ctx)
    return ctx


class _GatherSequence(torch.autograd.Function):
    """Local zig-zag rows ``[B, 2c, H, D]`` -> the whole sequence ``[B, S, H, D]`` on every rank; the backward pass sums
    the ranks' gradients of the whole sequence and keeps the local rows."""

    @staticmethod
    def forward(ctx, x: Tensor, world: int, rank: int, group):
        ctx.world, ctx.rank, ctx.group = world, rank, group
        parts = [torch.empty_like(x) for _ in range(world)]
        dist.all_gather(parts, x.contiguous(), group=group)
        return zigzag_merge(parts, dim=1)

    @staticmethod
    def backward(ctx, g: Tensor):
        g = g.contiguous().clone()
        dist.all_reduce(g, group=ctx.group)
        return zigzag_split(g, ctx.world, ctx.rank, dim=1), None, None, None


def _ring_attention_plain(q: Tensor, k: Tensor, v: Tensor, cp: CPContext, scale: float) -> Tensor:
    """Plain PyTorch statement of the sharded op (any device): gather K / V, mask by global positions."""
    b, two_c, hq, d = q.shape
    s = two_c * cp.world
    k_full = _GatherSequence.apply(k, cp.world, cp.rank, cp.group)
    v_full = _GatherSequence.apply(v, cp.world, cp.rank, cp.group)
    g = hq // k.size(2)
    kf, vf = k_full.repeat_interleave(g, dim=2), v_full.repeat_interleave(g, dim=2)
    q_pos = zigzag_positions(s, cp.world, cp.rank, device=q.device)
    mask = q_pos[:, None] >= torch.arange(s, device=q.device)[None, :]
    out = torch.nn.functional.scaled_dot_product_attention(q.transpose(1, 2), kf.transpose(1, 2), vf.transpose(1, 2),
                                                           attn_mask=mask, scale=scale)
    return out.transpose(1, 2)


# --------------------------------------------------------------------------- the op
def _gather_nccl(k: Tensor, v: Tensor, world: int, group) -> Tuple[Tensor, Tensor]:
    """all-gather + un-zig-zag: [B, 2c, H, D] per rank -> [B, S, H, D]."""
    b, two_c, h, d = k.shape
    c = two_c // 2
    local = torch.stack([k, v]).contiguous()                       # [2, B, 2c, H, D]
    gathered = torch.empty((world,) + local.shape, dtype=k.dtype, device=k.device)
    dist.all_gather_into_tensor(gathered, local, group=group)
    g = gathered.view(world, 2, b, 2, c, h, d)
    full = torch.empty(2, b, 2 * world, c, h, d, dtype=k.dtype, device=k.device)
    full[:, :, :world] = g[:, :, :, 0].permute(1, 2, 0, 3, 4, 5)
    full[:, :, world:] = g[:, :, :, 1].flip(0).permute(1, 2, 0, 3, 4, 5)
    full = full.view(2, b, 2 * world * c, h, d)
    return full[0], full[1]


def _scatter_nccl(dk_full: Tensor, dv_full: Tensor, world: int, group) -> Tuple[Tensor, Tensor]:
    """zig-zag + reduce-scatter: partial [B, S, H, D] -> summed local [B, 2c, H, D]."""
    b, s, h, d = dk_full.shape
    c = s // (2 * world)
    part = torch.stack([dk_full, dv_full]).view(2, b, 2 * world, c, h, d)
    send = torch.empty(world, 2, b, 2, c, h, d, dtype=dk_full.dtype, device=dk_full.device)
    send[:, :, :, 0] = part[:, :, :world].permute(2, 0, 1, 3, 4, 5)
    send[:, :, :, 1] = part[:, :, world:].flip(2).permute(2, 0, 1, 3, 4, 5)
    out = torch.empty(2, b, 2, c, h, d, dtype=torch.float32, device=dk_full.device)
    dist.reduce_scatter_tensor(out, send.float(), group=group)
    out = out.to(dk_full.dtype).view(2, b, 2 * c, h, d)
    return out[0], out[1]


class _RingAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q: Tensor, k: Tensor, v: Tensor, cp: CPContext, scale: float, comm: str):
        ops = torch.ops.astrai_b200
        b, two_c, hq, d = q.shape
        hkv, c, w, r = k.size(2), two_c // 2, cp.world, cp.rank
        row, s = hkv * d, 2 * cp.world * (two_c // 2)
        qf = q.contiguous().view(b * two_c, hq, d)
        if comm == "p2p":
            epoch = cp.next_epoch("fwd")
            src = cp.kv_source(b, c, row, epoch & 1)
            pair = src.tensor.view(2, b, two_c, hkv, d)
            pair[0].copy_(k)
            pair[1].copy_(v)
            k_full = torch.empty(b * s, hkv, d, dtype=q.dtype, device=q.device)
            v_full = torch.empty_like(k_full)
            out, lse = ops.cp_flash_fwd(qf, k_full, v_full, b, c, w, r, scale, src.peer_ptrs, cp.flags.peer_ptrs, 0, 1, epoch,
                                        cp.n_copy_ctas, cp.chunk_state, cp.timeout_s)
        else:
            kf, vf = _gather_nccl(k, v, w, cp.group)
            k_full, v_full = kf.reshape(b * s, hkv, d), vf.reshape(b * s, hkv, d)
            out, lse = ops.cp_flash_fwd(qf, k_full, v_full, b, c, w, r, scale, [], [], 0, 1, 0, 0, None, cp.timeout_s)
        ctx.save_for_backward(qf, k_full, v_full, out, lse)
        ctx.cp, ctx.scale, ctx.comm, ctx.shape = cp, scale, comm, (b, two_c, hq, hkv, d)
        return out.view(b, two_c, hq, d)

    @staticmethod
    def backward(ctx, dout: Tensor):
        ops = torch.ops.astrai_b200
        qf, k_full, v_full, out, lse = ctx.saved_tensors
        cp, (b, two_c, hq, hkv, d) = ctx.cp, ctx.shape
        c, w, r, row = two_c // 2, cp.world, cp.rank, hkv * d
        do = dout.contiguous().view(b * two_c, hq, d)
        if ctx.comm == "p2p":
            epoch = cp.next_epoch("bwd")
            stage = cp.stage(b, c, row, epoch & 1)
            dq, _, _ = ops.cp_flash_bwd(qf, k_full, v_full, out, do, lse, b, c, w, r, ctx.scale, stage.peer_ptrs,
                                        cp.flags.peer_ptrs, 0, 1, epoch, cp.tile_counter, cp.timeout_s)
            dk = torch.empty(b * two_c, hkv, d, dtype=qf.dtype, device=qf.device)
            dv = torch.empty_like(dk)
            ops.cp_dkv_reduce(dk, dv, b, c, w, r, stage.peer_ptrs, cp.flags.peer_ptrs, 0, 1, epoch, cp.timeout_s)
            dk, dv = dk.view(b, two_c, hkv, d), dv.view(b, two_c, hkv, d)
        else:
            dq, dk_full, dv_full = ops.cp_flash_bwd(qf, k_full, v_full, out, do, lse, b, c, w, r, ctx.scale, [], [], 0, 1, 0,
                                                    None, cp.timeout_s)
            s = 2 * w * c
            dk, dv = _scatter_nccl(dk_full.view(b, s, hkv, d), dv_full.view(b, s, hkv, d), w, cp.group)
        return dq.view(b, two_c, hq, d), dk, dv, None, None, None


def supported(q: Tensor, k: Tensor, v: Tensor) -> bool:
    """Shapes the fused kernels take: bf16 on CUDA, head_dim 64 / 128, local rows = two chunks of whole 128-key tiles."""
    return (q.is_cuda and q.dtype == torch.bfloat16 and k.dtype == v.dtype == torch.bfloat16 and q.dim() == 4
            and q.size(3) in (64, 128) and q.size(1) % (2 * TILE) == 0 and k.shape == v.shape
            and k.size(1) == q.size(1) and q.size(2) % k.size(2) == 0)


def ring_attention(q: Tensor, k: Tensor, v: Tensor, scale: Optional[float] = None, ctx: Optional[CPContext] = None,
                   comm: str = "p2p") -> Tensor:
    """Causal attention of the zig-zag-sharded sequence.  q [B, 2c, Hq, D], k / v [B, 2c, Hkv, D] local rows -> [B, 2c, Hq, D].

    Collective over the context-parallel group: every rank calls it with its own rows, in the same order.
    """
    cp = ctx or get_context()
    if cp is None:
        raise RuntimeError("ring_attention needs a context: call init_context_parallel() first")
    if comm not in ("p2p", "nccl"):
        raise ValueError(f"unknown comm {comm!r}")
    if not q.is_cuda or cp.arena is None and not supported(q, k, v):
        return _ring_attention_plain(q, k, v, cp, float(scale) if scale is not None else 1.0 / math.sqrt(q.size(3)))
    if cp.arena is None:
        comm = "nccl"
    if not supported(q, k, v):
        raise ValueError("ring_attention: bf16 CUDA tensors [B, 2c, H, D] with D in {64, 128} and c a multiple of 128")
    scale = float(scale) if scale is not None else 1.0 / math.sqrt(q.size(3))
    return _RingAttention.apply(q, k, v, cp, scale, comm)


def ring_attention_reference(q_parts: List[Tensor], k_parts: List[Tensor], v_parts: List[Tensor],
                             scale: Optional[float] = None) -> List[Tensor]:
    """Plain PyTorch restatement over every rank's rows at once (tests, CPU): merge, causal attention, split."""
    world = len(q_parts)
    q, k, v = (zigzag_merge(p, dim=1).float() for p in (q_parts, k_parts, v_parts))
    g = q.size(2) // k.size(2)
    k, v = k.repeat_interleave(g, dim=2), v.repeat_interleave(g, dim=2)
    out = torch.nn.functional.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2),
                                                           is_causal=True, scale=scale).transpose(1, 2)
    return [zigzag_split(out, world, r, dim=1) for r in range(world)]
