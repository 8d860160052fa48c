"""Symmetric memory: one arena per rank, mapped into every rank of the node.

The fused compute+collective kernels address their peers' buffers directly over NVLink (plain loads / stores) or
through the NVSwitch multicast mapping of the same arena (``multimem.*``).  The arena is created once with
``torch.distributed._symmetric_memory`` (CUDA VMM allocation + handle exchange over the process group, which is the
only role NCCL / the store plays here) and carved into sub-buffers; a sub-buffer's address on rank ``r`` is
``arena_ptr[r] + offset``, identical offsets everywhere.

The reference has no counterpart: its only transport is ``torch.distributed`` collectives
(``astrai/parallel/setup.py:44-90``).

:class:`LocalArena` gives the same interface inside ONE process (several "ranks" as slices of one allocation).  It is
what single-GPU tests use to run every rank's kernel one after the other with the flags preset - kernels of
different ranks that wait for one another must never be launched on the same GPU.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.distributed as dist

FLAG_KINDS = 8        # independent flag planes ([kind][8 ranks][max_units] int32 per rank)
MAX_RANKS = 8
KIND_GRADS_READY, KIND_PARAMS_WRITTEN, KIND_TP_AG, KIND_TP_RS, KIND_CP, KIND_EP, KIND_CP_DKV = 0, 1, 2, 3, 4, 5, 6


@dataclass
class SymmBuffer:
    """A tensor view of this rank's part plus the device addresses of the same bytes on every rank."""

    tensor: torch.Tensor
    offset: int            # bytes from the arena base
    peer_ptrs: List[int]
    mc_ptr: int            # 0 when the arena has no multicast mapping

    def ptrs_at(self, elem_offset: int = 0) -> List[int]:
        b = elem_offset * self.tensor.element_size()
        return [p + b for p in self.peer_ptrs]


class _ArenaBase:
    rank: int
    world_size: int

    def _carve(self, nbytes: int, align: int = 256) -> int:
        off = -(-self._used // align) * align
        if off + nbytes > self.capacity:
            raise RuntimeError(f"symmetric arena exhausted: need {off + nbytes} bytes, capacity {self.capacity}")
        self._used = off + nbytes
        return off

    def alloc(self, numel: int, dtype: torch.dtype, zero: bool = True) -> SymmBuffer:
        nbytes = numel * torch.empty((), dtype=dtype).element_size()
        off = self._carve(nbytes)
        # A tensor of its own over the arena's storage (not a view of it): views of one base share a version
        # counter, and an in-place update of one flat buffer would then invalidate autograd's saved views of another.
        base = self._local_bytes()
        item = nbytes // max(numel, 1) if numel else 1
        t = torch.empty(0, dtype=dtype, device=base.device).set_(
            base.untyped_storage(), (base.storage_offset() + off) // item, (numel,), (1,))
        if zero:
            t.zero_()
        return SymmBuffer(t, off, [p + off for p in self._base_ptrs()], (self._mc_base() + off) if self._mc_base() else 0)

    def alloc_flags(self, max_units: int) -> SymmBuffer:
        return self.alloc(FLAG_KINDS * MAX_RANKS * max_units, torch.int32, zero=True)


class SymmetricArena(_ArenaBase):
    """``capacity`` bytes on this rank's GPU, reachable from every rank of ``group`` (collective constructor)."""

    def __init__(self, capacity: int, device: Optional[torch.device] = None, group=None):
        import torch.distributed._symmetric_memory as symm_mem

        if not dist.is_initialized():
            raise RuntimeError("SymmetricArena needs an initialised process group")
        self.group = group if group is not None else dist.group.WORLD
        self.rank, self.world_size = dist.get_rank(self.group), dist.get_world_size(self.group)
        if self.world_size > MAX_RANKS:
            raise RuntimeError("peer-memory kernels address at most 8 ranks (one NVSwitch domain)")
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.capacity = -(-int(capacity) // (2 << 20)) * (2 << 20)
        self._buf = symm_mem.empty(self.capacity, dtype=torch.uint8, device=self.device)
        self._handle = symm_mem.rendezvous(self._buf, self.group)
        self._ptrs = [int(p) for p in self._handle.buffer_ptrs]
        try:
            self._mc = int(self._handle.multicast_ptr) if self._handle.has_multicast_support else 0
        except Exception:  # noqa: BLE001 - multicast is optional
            self._mc = 0
        self._used = 0

    def _local_bytes(self) -> torch.Tensor:
        return self._buf

    def _base_ptrs(self) -> List[int]:
        return self._ptrs

    def _mc_base(self) -> int:
        return self._mc

    @property
    def has_multicast(self) -> bool:
        return self._mc != 0

    def barrier(self):
        """Device-side barrier of the arena's ranks on the current stream (signal pads of the handle)."""
        self._handle.barrier(channel=0)


class LocalArena(_ArenaBase):
    """``world_size`` emulated ranks inside one process; ``view(rank)`` selects whose part ``alloc`` returns."""

    def __init__(self, capacity: int, world_size: int, device):
        self.capacity = -(-int(capacity) // 256) * 256
        self.world_size, self.rank = world_size, 0
        self._all = torch.zeros(world_size, self.capacity, dtype=torch.uint8, device=device)
        self._used = 0

    def view(self, rank: int) -> "LocalArena":
        other = object.__new__(LocalArena)
        other.__dict__.update(self.__dict__)
        other.rank = rank
        other._used = 0
        return other

    def _local_bytes(self) -> torch.Tensor:
        return self._all[self.rank]

    def _base_ptrs(self) -> List[int]:
        return [self._all[r].data_ptr() for r in range(self.world_size)]

    def _mc_base(self) -> int:
        return 0

    has_multicast = False

    def barrier(self):
        pass
