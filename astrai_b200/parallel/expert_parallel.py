"""Expert-parallel mixture of experts: every rank owns ``E / W`` experts; tokens travel to their experts and back over
NVLink inside the expert GEMMs.

Per layer call and rank (all on the device, no host round trip, no collective call):

1. the local router picks ``top_k`` experts per token (``ops/moe.py::route``);
2. ``ep_push_counts`` / ``ep_plan`` (``ops/csrc/moe_ep.cu``) exchange the per-expert counts through peer memory, lay
   out every rank's padded expert segments and enter each ``(token, choice)`` into the row table of the expert's owner;
3. the gate|up grouped GEMM *pulls* its rows: copy CTAs inside the launch gather each 128-row tile from the peers'
   activations with bulk copies while the GEMM CTAs work on the tiles that have landed (dispatch all-to-all fused into
   the GEMM, ``ops/csrc/gemm_grouped.cu``);
4. SwiGLU on the sorted rows, then the down grouped GEMM whose epilogue *pushes* every output row into the memory of
   the rank that owns the token (combine all-to-all fused into the GEMM);
5. the token's owner sums its ``top_k`` returned rows with the router weights.

The backward pass is the mirror image: the gradient rows are pulled by the down-projection dgrad GEMM and pushed back by
the gate|up dgrad GEMM; weight gradients are local grouped GEMMs over the sorted rows.

The reference computes its MoE on one device with a Python loop over experts
(``astrai/model/components/mlp.py:95-172``) and has no expert parallelism.
"""

from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch
from torch import Tensor, nn

from astrai_b200.parallel import symm

TILE = 128
MAX_UNITS = 8
U_COUNTS, U_TABLE, U_Y, U_DY, U_DX = 0, 1, 2, 3, 4


class EPContext:
    """Per-process state: arena, flags, epochs, parity-double-buffered exchange buffers."""

    def __init__(self, arena, rank: int, world: int, timeout_s: float = 60.0, n_copy_ctas: int = 16, group=None):
        if not 2 <= world <= symm.MAX_RANKS:
            raise ValueError(f"expert parallel world size must be in 2..{symm.MAX_RANKS}")
        self.arena, self.rank, self.world, self.group = arena, rank, world, group
        self.timeout_s, self.n_copy_ctas = float(timeout_s), int(n_copy_ctas)
        self.flags = arena.alloc_flags(MAX_UNITS)
        self._pool: Dict[Tuple, symm.SymmBuffer] = {}
        self._epoch = {"fwd": 0, "bwd": 0}
        dev = self.flags.tensor.device
        self.done_counter = torch.zeros(1, dtype=torch.int32, device=dev)
        self._tile_flags: Dict[Tuple[str, int], Tensor] = {}
        self.last_dropped: Optional[Tensor] = None  # pairs dropped by the capacity limit in the latest call (0-d tensor)

    # Every call has an all-to-all synchronisation of its own (the counts exchange / the gradient announcement), so a
    # buffer of call n is free again when call n + 2 starts: two parities are enough.  Allocation order is the same on
    # every rank because the same model code runs everywhere.
    def buf(self, kind: str, numel: int, dtype: torch.dtype, parity: int) -> symm.SymmBuffer:
        key = (kind, numel, dtype, parity)
        if key not in self._pool:
            self._pool[key] = self.arena.alloc(numel, dtype, zero=False)
        return self._pool[key]

    def tile_flags(self, direction: str, tiles: int) -> Tensor:
        key = (direction, tiles)
        if key not in self._tile_flags:
            self._tile_flags[key] = torch.zeros(tiles, dtype=torch.int32, device=self.flags.tensor.device)
        return self._tile_flags[key]

    def next_epoch(self, direction: str) -> int:
        self._epoch[direction] += 1
        return self._epoch[direction]


_CTX: Optional[EPContext] = None


def set_context(ctx: Optional[EPContext]):
    global _CTX
    _CTX = ctx


def get_context() -> Optional[EPContext]:
    return _CTX


def row_capacity(tokens: int, top_k: int, world: int, local_experts: int, capacity_factor: Optional[float] = None) -> int:
    """Rows of the sorted buffer on one rank.  Without a capacity factor the worst case (every pair of every rank lands
    here) is reserved; with one, ``capacity_factor x`` the balanced share, and a step that exceeds it raises."""
    pairs = tokens * top_k * world if capacity_factor is None else int(tokens * top_k * capacity_factor)
    return -(-pairs // TILE) * TILE + local_experts * TILE


def limit_rows_per_rank(idx: Tensor, weights: Tensor, n_experts: int, world: int, capacity_factor: float):
    """Token dropping for a capacity-bounded exchange, without a host synchronisation.

    Of this rank's ``T x k`` (token, choice) pairs at most ``floor(capacity_factor * T * k / world)`` may go to the experts of
    any one rank; with every sender keeping to that, no receiver's buffer of ``capacity_factor * T * k`` rows can overflow.
    Pairs beyond a destination's limit (in token order) are *dropped*: their routing weight becomes 0 (so they add
    nothing to the output and receive no gradient) and they are re-addressed to the first expert of a rank that still has
    room, because the exchange moves a dense ``[T, k]`` table.  Returns ``(idx, weights, counts [E] int32, dropped)`` with
    ``dropped`` a 0-d tensor (the number of dropped pairs, for logging); kept pairs are returned unchanged.
    Needs ``capacity_factor >= 1`` (otherwise the pairs cannot all be placed)."""
    if capacity_factor < 1.0:
        raise ValueError("capacity_factor must be at least 1: every pair has to be placed somewhere")
    t, k = idx.shape
    local = n_experts // world
    cap = int(capacity_factor * t * k) // world
    flat = idx.reshape(-1).long()
    dst = flat // local                                                            # destination rank of every pair
    onehot = torch.nn.functional.one_hot(dst, world)                               # [T*k, W]
    pos = (onehot.cumsum(0) * onehot).sum(1) - 1                                   # position among the pairs of its rank
    over = pos >= cap
    sent = onehot.sum(0)                                                           # pairs per destination before the limit
    room = (cap - sent).clamp(min=0)                                               # free rows per destination
    # the j-th dropped pair takes the j-th free row, destinations in rank order
    j = over.long().cumsum(0) - 1
    new_dst = torch.searchsorted(room.cumsum(0), j.clamp(min=0), right=True).clamp(max=world - 1)
    new_flat = torch.where(over, new_dst * local, flat)
    keep = (~over).to(weights.dtype).view(t, k)
    counts = torch.bincount(new_flat, minlength=n_experts).to(torch.int32)
    return new_flat.view(t, k).to(idx.dtype), weights * keep, counts, over.sum()


def arena_bytes_for(tokens: int, hidden: int, top_k: int, world: int, n_experts: int,
                    capacity_factor: Optional[float] = None) -> int:
    rows = tokens * top_k
    cap = row_capacity(tokens, top_k, world, n_experts // world, capacity_factor)
    per_parity = tokens * hidden * 2 + 3 * rows * hidden * 2 + world * n_experts * 4 + cap * 4
    return 2 * per_parity + (1 << 20)


def init_expert_parallel(arena_bytes: int, timeout_s: float = 60.0, group=None, n_copy_ctas: int = 16) -> EPContext:
    """Collective: create the symmetric arena of the expert-parallel group and install the context."""
    arena = symm.SymmetricArena(arena_bytes, group=group)
    ctx = EPContext(arena, arena.rank, arena.world_size, timeout_s=timeout_s, n_copy_ctas=n_copy_ctas, group=group)
    set_context(ctx)
    return ctx


def _identity_slots(tokens: int, k: int, device) -> Tensor:
    return torch.arange(tokens * k, dtype=torch.int32, device=device).view(tokens, k)


# The pass is written as phases so that a single-GPU test can run phase i of every emulated rank before phase i + 1 of
# any (kernels of different ranks that wait for one another must not share a GPU); _EPExpertsFn runs them back to back.
class _State:
    pass


def _fwd_push(ep: EPContext, x: Tensor, idx: Tensor, counts: Tensor, r_cap: int) -> _State:
    ops = torch.ops.astrai_b200
    st = _State()
    st.ep, st.r_cap, st.t, st.h, st.k = ep, r_cap, x.shape[0], x.shape[1], idx.shape[1]
    st.n_experts, st.dtype, st.device = counts.numel(), x.dtype, x.device
    st.fe = ep.next_epoch("fwd")
    par = st.fe & 1
    st.x_src = ep.buf("x", st.t * st.h, x.dtype, par)
    st.x_src.tensor.view(st.t, st.h).copy_(x)
    st.counts_all = ep.buf("counts", ep.world * st.n_experts, torch.int32, par)
    st.rows = ep.buf("rows", r_cap, torch.int32, par)
    st.y_slots = ep.buf("y", st.t * st.k * st.h, x.dtype, par)
    st.idx = idx.contiguous()
    ops.ep_push_counts(counts, st.counts_all.peer_ptrs, st.rows.tensor, ep.flags.peer_ptrs, ep.rank, U_COUNTS, MAX_UNITS, st.fe)
    return st


def _fwd_plan(st: _State):
    ep = st.ep
    st.offsets, st.tile_expert, st.total = torch.ops.astrai_b200.ep_plan(
        st.idx, st.counts_all.tensor, st.rows.peer_ptrs, st.n_experts, st.r_cap, ep.flags.peer_ptrs, ep.rank, U_COUNTS, U_TABLE,
        MAX_UNITS, st.fe, ep.timeout_s)


def _fwd_experts(st: _State, w_gate_up: Tensor, w_down: Tensor):
    ops, ep = torch.ops.astrai_b200, st.ep
    fl = ep.flags.peer_ptrs
    st.x_sorted = torch.empty(st.r_cap, st.h, dtype=st.dtype, device=st.device)
    st.hgu = ops.grouped_gemm_rows_ep(st.x_sorted, w_gate_up, True, st.tile_expert, st.rows.tensor, ep.rank, st.x_src.peer_ptrs, st.k,
                                      ep.tile_flags("fwd", st.r_cap // TILE), ep.n_copy_ctas, [], None, fl, -1, U_TABLE, 0,
                                      MAX_UNITS, st.fe, ep.timeout_s)
    st.row_peer = st.rows.tensor.clone()  # complete once the gather has run; the exchange buffer is reused two calls on
    f = st.hgu.shape[1] // 2
    act = ops.swiglu_fwd(st.hgu[:, :f], st.hgu[:, f:])
    ops.grouped_gemm_rows_ep(act, w_down, True, st.tile_expert, st.row_peer, ep.rank, [], 1, None, 0, st.y_slots.peer_ptrs,
                             ep.done_counter, fl, -1, 0, U_Y, MAX_UNITS, st.fe, ep.timeout_s)


def _fwd_combine(st: _State, weights: Tensor) -> Tensor:
    ops, ep = torch.ops.astrai_b200, st.ep
    ops.comm_wait_flags_(ep.flags.tensor, symm.KIND_EP, ep.world, -1, U_Y, MAX_UNITS, st.fe, ep.timeout_s)
    st.y = st.y_slots.tensor.view(st.t * st.k, st.h).clone()
    st.slots = _identity_slots(st.t, st.k, st.device)
    return ops.moe_combine(st.y, st.slots, weights.contiguous())


def _bwd_prepare(st: _State, dout: Tensor, weights: Tensor) -> Tensor:
    ops, ep = torch.ops.astrai_b200, st.ep
    st.be = ep.next_epoch("bwd")
    par = st.be & 1
    dy, dweights = ops.moe_combine_bwd(dout.contiguous(), st.y, st.slots, weights.contiguous())
    st.dy_slots = ep.buf("dy", st.t * st.k * st.h, st.dtype, par)
    st.dx_slots = ep.buf("dx", st.t * st.k * st.h, st.dtype, par)
    st.dy_slots.tensor.view(st.t * st.k, st.h).copy_(dy)
    return dweights


def _bwd_experts(st: _State, w_gate_up: Tensor, w_down: Tensor):
    ops, ep = torch.ops.astrai_b200, st.ep
    fl = ep.flags.peer_ptrs
    dy_sorted = torch.empty(st.r_cap, st.h, dtype=st.dtype, device=st.device)
    dact = ops.grouped_gemm_rows_ep(dy_sorted, w_down, False, st.tile_expert, st.row_peer, ep.rank, st.dy_slots.peer_ptrs, 1,
                                    ep.tile_flags("bwd", st.r_cap // TILE), ep.n_copy_ctas, [], None, fl, U_DY, U_DY, 0,
                                    MAX_UNITS, st.be, ep.timeout_s)
    f = st.hgu.shape[1] // 2
    act = ops.swiglu_fwd(st.hgu[:, :f], st.hgu[:, f:])
    dw_down = ops.grouped_gemm_wgrad(dy_sorted, act, st.offsets, False)
    dh = ops.swiglu_bwd(dact, st.hgu[:, :f], st.hgu[:, f:])  # [rows, 2F]: d gate | d up
    ops.grouped_gemm_rows_ep(dh, w_gate_up, False, st.tile_expert, st.row_peer, ep.rank, [], 1, None, 0, st.dx_slots.peer_ptrs,
                             ep.done_counter, fl, -1, 0, U_DX, MAX_UNITS, st.be, ep.timeout_s)
    dw_gate_up = ops.grouped_gemm_wgrad(dh, st.x_sorted, st.offsets, False)
    return dw_gate_up, dw_down


def _bwd_finish(st: _State) -> Tensor:
    ops, ep = torch.ops.astrai_b200, st.ep
    ops.comm_wait_flags_(ep.flags.tensor, symm.KIND_EP, ep.world, -1, U_DX, MAX_UNITS, st.be, ep.timeout_s)
    return ops.moe_combine(st.dx_slots.tensor.view(st.t * st.k, st.h), st.slots, None)


class _EPExpertsFn(torch.autograd.Function):
    """x [T, H], idx [T, K], weights [T, K], counts [E] -> sum_k weights * expert_k(x): the routed experts of all ranks."""

    @staticmethod
    def forward(ctx, x: Tensor, idx: Tensor, weights: Tensor, counts: Tensor, w_gate_up: Tensor, w_down: Tensor,
                ep: EPContext, r_cap: int):
        st = _fwd_push(ep, x, idx, counts, r_cap)
        _fwd_plan(st)
        _fwd_experts(st, w_gate_up, w_down)
        out = _fwd_combine(st, weights)
        ctx.save_for_backward(weights, w_gate_up, w_down)
        ctx.st = st
        return out

    @staticmethod
    def backward(ctx, dout: Tensor):
        weights, w_gate_up, w_down = ctx.saved_tensors
        st = ctx.st
        dweights = _bwd_prepare(st, dout, weights)
        dw_gate_up, dw_down = _bwd_experts(st, w_gate_up, w_down)
        dx = _bwd_finish(st)
        return dx, None, dweights.to(weights.dtype), None, dw_gate_up, dw_down, None, None


def ep_experts(x: Tensor, idx: Tensor, weights: Tensor, counts: Tensor, w_gate_up: Tensor, w_down: Tensor,
               ctx: Optional[EPContext] = None, capacity_factor: Optional[float] = 2.0) -> Tensor:
    """Routed-expert output for the local tokens; collective over the expert-parallel group.

    ``w_gate_up`` ``[E / W, 2F, H]`` and ``w_down`` ``[E / W, H, F]`` are this rank's experts; ``idx`` / ``counts`` use
    global expert numbers (rank ``d`` owns ``[d * E / W, (d + 1) * E / W)``).  The sorted buffers hold
    ``capacity_factor`` times the balanced share of rows (``None``: the worst case, every pair of every rank).  With a
    capacity factor every sender keeps to its share of each receiver's buffer (:func:`limit_rows_per_rank`: pairs beyond
    it are dropped, i.e. contribute nothing), so a receiver cannot overflow; error 72 of the kernel status word remains
    as the check behind that.
    """
    ep = ctx or get_context()
    if ep is None:
        raise RuntimeError("ep_experts needs a context: call init_expert_parallel() first")
    n_experts = counts.numel()
    if n_experts % ep.world or w_gate_up.shape[0] != n_experts // ep.world:
        raise ValueError("experts must divide evenly over the ranks and the weights hold this rank's share")
    if not (x.is_cuda and x.dtype == torch.bfloat16 and x.shape[1] % 64 == 0 and w_gate_up.shape[1] % 64 == 0):
        raise ValueError("ep_experts: bf16 CUDA activations with hidden and intermediate sizes that are multiples of 64")
    r_cap = row_capacity(x.shape[0], idx.shape[1], ep.world, n_experts // ep.world, capacity_factor)
    if capacity_factor is not None and ep.world > 1:
        idx, weights, counts, ep.last_dropped = limit_rows_per_rank(idx, weights, n_experts, ep.world, capacity_factor)
    return _EPExpertsFn.apply(x.contiguous(), idx, weights, counts, w_gate_up, w_down, ep, r_cap)


class EPMoE(nn.Module):
    """A routed mixture of experts whose experts are sharded over the expert-parallel group.

    Same routing as ``models/ffn.py::DeepSeekMoE`` (softmax router, top-k, optional renormalisation); the experts'
    weights are stored stacked - ``gate_up`` ``[E / W, 2F, H]`` and ``down`` ``[E / W, H, F]`` - so the grouped GEMMs read
    them in place.  The router is replicated (its gradient must be all-reduced by the data-parallel wrapper like any
    replicated parameter); the expert weights are not.
    """

    def __init__(self, dim: int, moe_inter_dim: int, n_experts: int, top_k: int, ep_size: int, ep_rank: int,
                 norm_topk_prob: bool = True, init_std: float = 0.02, capacity_factor: Optional[float] = 2.0, dtype=None,
                 device=None):
        super().__init__()
        if n_experts % ep_size:
            raise ValueError("n_experts must be a multiple of ep_size")
        self.dim, self.inter, self.n_experts, self.top_k = dim, moe_inter_dim, n_experts, top_k
        self.ep_size, self.ep_rank, self.norm_topk_prob = ep_size, ep_rank, norm_topk_prob
        self.capacity_factor = capacity_factor
        local = n_experts // ep_size
        kw = {"dtype": dtype, "device": device}
        self.router = nn.Parameter(torch.empty(n_experts, dim, **kw).normal_(0, init_std))
        self.gate_up = nn.Parameter(torch.empty(local, 2 * moe_inter_dim, dim, **kw).normal_(0, init_std))
        self.down = nn.Parameter(torch.empty(local, dim, moe_inter_dim, **kw).normal_(0, init_std))

    @staticmethod
    def shard(full: Tensor, ep_size: int, ep_rank: int) -> Tensor:
        """This rank's slice of a tensor stacked over all experts."""
        local = full.shape[0] // ep_size
        return full[ep_rank * local:(ep_rank + 1) * local]

    def forward(self, x: Tensor, ctx: Optional[EPContext] = None) -> Tensor:
        from astrai_b200.ops import functional as F
        from astrai_b200.ops import moe

        shape = x.shape
        flat = x.reshape(-1, shape[-1])
        logits = F.linear(flat, self.router)
        _probs, idx, weights, counts, _psum = moe.route(logits, self.top_k, self.norm_topk_prob)
        out = ep_experts(flat, idx, weights, counts, self.gate_up, self.down, ctx=ctx, capacity_factor=self.capacity_factor)
        return out.view(shape)


def moe_reference(x_parts, router: Tensor, gate_up: Tensor, down: Tensor, top_k: int, norm_topk_prob: bool = True):
    """Plain PyTorch fp32 restatement over every rank's tokens with ALL experts' stacked weights (tests, CPU)."""
    outs = []
    f = gate_up.shape[1] // 2
    for x in x_parts:
        xf = x.float()
        probs = torch.softmax(xf @ router.float().t(), dim=-1).to(x.dtype).float()
        w, idx = torch.topk(probs, top_k, dim=-1)
        if norm_topk_prob:
            w = w / w.sum(-1, keepdim=True)
        w = w.to(x.dtype).float()
        out = torch.zeros_like(xf)
        for e in range(gate_up.shape[0]):
            sel = (idx == e)
            rows = sel.any(-1).nonzero().flatten()
            if rows.numel() == 0:
                continue
            hgu = xf[rows] @ gate_up[e].float().t()
            act = torch.nn.functional.silu(hgu[:, :f]) * hgu[:, f:]
            out[rows] += (w[rows] * sel[rows]).sum(-1, keepdim=True) * (act @ down[e].float().t())
        outs.append(out)
    return outs


# --------------------------------------------------------------------------- collective arm (baseline, and the CPU path)
def _supports_all_to_all(group) -> bool:
    import torch.distributed as dist

    return dist.get_backend(group) != "gloo"


class _AllToAllRows(torch.autograd.Function):
    """Rows ``x`` cut into one segment per destination rank (``send``) travel to their ranks; the result is the segments
    received from every rank in rank order (``recv``).  The backward pass is the same exchange with the roles swapped."""

    @staticmethod
    def forward(ctx, x: Tensor, send, recv, group, seg_cap: int):
        ctx.send, ctx.recv, ctx.group, ctx.seg_cap = list(send), list(recv), group, seg_cap
        return _exchange_rows(x, ctx.send, ctx.recv, group, seg_cap)

    @staticmethod
    def backward(ctx, g: Tensor):
        return _exchange_rows(g.contiguous(), ctx.recv, ctx.send, ctx.group, ctx.seg_cap), None, None, None, None


def _exchange_rows(x: Tensor, send, recv, group, seg_cap: int) -> Tensor:
    import torch.distributed as dist

    out = torch.empty((sum(recv),) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    if _supports_all_to_all(group):
        dist.all_to_all_single(out, x.contiguous(), output_split_sizes=list(recv), input_split_sizes=list(send), group=group)
        return out
    # Gloo has no all-to-all: every rank publishes its padded segments and each reader cuts out what was meant for it.
    world, me = dist.get_world_size(group), dist.get_rank(group)
    padded = torch.zeros((world, seg_cap) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    at = 0
    for d, n in enumerate(send):
        padded[d, :n] = x[at:at + n]
        at += n
    everything = torch.empty((world * world,) + tuple(padded.shape[1:]), dtype=x.dtype, device=x.device)
    dist.all_gather_into_tensor(everything, padded, group=group)
    everything = everything.view((world,) + tuple(padded.shape))
    at = 0
    for s, n in enumerate(recv):
        out[at:at + n] = everything[s, me, :n]
        at += n
    return out


def ep_experts_collective(x: Tensor, idx: Tensor, weights: Tensor, counts: Tensor, w_gate_up: Tensor, w_down: Tensor,
                          group=None) -> Tensor:
    """The same function as :func:`ep_experts` built from library collectives: counts all-gather, token all-to-all,
    one GEMM pair per local expert, all-to-all back, weighted sum.  Split sizes are read back to the host (one sync per
    call), which the fused path avoids.  It is the arm the fused kernels are measured against, and the CPU path."""
    import torch.distributed as dist
    from astrai_b200 import ops

    world, me = dist.get_world_size(group), dist.get_rank(group)
    t, h = x.shape
    k, n_experts = idx.shape[1], counts.numel()
    local = n_experts // world
    all_counts = torch.empty(world * n_experts, dtype=counts.dtype, device=counts.device)
    dist.all_gather_into_tensor(all_counts, counts.contiguous(), group=group)
    table = all_counts.view(world, world, local).cpu()               # [source rank, owner rank, local expert]
    send = table[me].sum(-1).tolist()                                # rows this rank sends to each owner
    recv = table[:, me].sum(-1).tolist()                             # rows this rank receives from each source
    seg_cap = int(table.sum(-1).max())
    order = torch.argsort(idx.reshape(-1), stable=True)              # (token, choice) pairs sorted by global expert
    token_of = order // k
    rows = _AllToAllRows.apply(x[token_of], send, recv, group, seg_cap)  # grouped by source rank, then by expert
    mine = table[:, me]                                              # [source, local expert] row counts held here
    seg_start = torch.zeros(world, local, dtype=torch.long)
    flat_sizes = mine.reshape(-1).long()
    seg_start.view(-1)[1:] = torch.cumsum(flat_sizes, 0)[:-1]
    by_expert = [torch.cat([torch.arange(int(seg_start[s, e]), int(seg_start[s, e] + mine[s, e])) for s in range(world)])
                 for e in range(local)]
    perm = torch.cat(by_expert).to(x.device) if by_expert else torch.empty(0, dtype=torch.long, device=x.device)
    sorted_rows = rows[perm]
    outs, at = [], 0
    f = w_gate_up.shape[1] // 2
    for e in range(local):
        n = int(mine[:, e].sum())
        seg = sorted_rows[at:at + n]
        at += n
        if n == 0:
            outs.append(seg.new_zeros((0, h)))
            continue
        hgu = ops.linear(seg, w_gate_up[e])
        outs.append(ops.linear(ops.swiglu(hgu[:, :f], hgu[:, f:]), w_down[e]))
    y_sorted = torch.cat(outs) if outs else sorted_rows
    inv = torch.empty_like(perm)
    inv[perm] = torch.arange(perm.numel(), device=perm.device)
    y = _AllToAllRows.apply(y_sorted[inv], recv, send, group, seg_cap)  # back in this rank's expert-sorted pair order
    y = y * weights.reshape(-1, 1)[order].to(y.dtype)
    return torch.zeros_like(x).index_add(0, token_of, y)


class EPExperts(nn.Module):
    """This rank's routed experts of one MoE layer, stacked: ``gate_up [E/W, 2F, H]`` and ``down [E/W, H, F]``.

    Built from the ``routed_experts`` list of a :class:`~astrai_b200.models.ffn.DeepSeekMoE` (whose place it takes under
    the same attribute name) by the expert-parallel executor; ``comm="p2p"`` runs the fused peer-memory kernels,
    ``"nccl"`` the collective arm."""

    def __init__(self, experts, ep_size: int, ep_rank: int, comm: str = "p2p", group=None,
                 capacity_factor: Optional[float] = 2.0):
        super().__init__()
        n = len(experts)
        if n % ep_size:
            raise ValueError(f"{n} routed experts do not divide over {ep_size} ranks")
        self.n_experts, self.ep_size, self.ep_rank, self.comm, self.group = n, ep_size, ep_rank, comm, group
        self.capacity_factor = capacity_factor
        local = n // ep_size
        mine = [experts[i] for i in range(ep_rank * local, (ep_rank + 1) * local)]
        self.gate_up = nn.Parameter(torch.stack([torch.cat([m.gate.weight, m.up.weight], dim=0) for m in mine]).detach().clone())
        self.down = nn.Parameter(torch.stack([m.down.weight for m in mine]).detach().clone())

    def forward(self, x: Tensor, idx: Tensor, weights: Tensor, counts: Tensor) -> Tensor:
        if self.comm == "p2p" and x.is_cuda and get_context() is not None:
            return ep_experts(x, idx, weights, counts.int(), self.gate_up, self.down, capacity_factor=self.capacity_factor)
        return ep_experts_collective(x, idx, weights, counts, self.gate_up, self.down, group=self.group)

    def unstacked(self, prefix: str, gate_up: Tensor, down: Tensor) -> Dict[str, Tensor]:
        """Reference checkpoint keys (``<prefix>.<j>.{gate,up,down}.weight``) for stacked tensors of ALL experts."""
        f = gate_up.shape[1] // 2
        out = {}
        for j in range(gate_up.shape[0]):
            out[f"{prefix}.{j}.gate.weight"] = gate_up[j, :f]
            out[f"{prefix}.{j}.up.weight"] = gate_up[j, f:]
            out[f"{prefix}.{j}.down.weight"] = down[j]
        return out
