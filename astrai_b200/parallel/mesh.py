"""Two-level rank layout for the model-parallel training modes.

The ``W`` ranks of a job are cut into blocks of ``mp_size`` consecutive ranks.  A block is one *model-parallel group*
(tensor-, context- or expert-parallel: its ranks hold parts of one model replica, or of one sequence, and talk to one
another in every forward pass, so a block never spans two NVSwitch domains).  Ranks that have the same position in
their blocks form a *data-parallel group* (they hold the same part of different replicas and only exchange gradients).

    world 8, mp_size 4:   model-parallel groups {0,1,2,3} {4,5,6,7};   data-parallel groups {0,4} {1,5} {2,6} {3,7}

The reference has one WORLD group and nothing else (``astrai/parallel/setup.py:44-90``).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, List, Optional

import torch.distributed as dist


@dataclass
class ParallelMesh:
    world: int
    rank: int
    mp_size: int
    mp_group: Any = None   # None: the group is WORLD (mp_size == world) or there is no process group at all
    dp_group: Any = None   # None: every data-parallel group has one member (mp_size == world) or it is WORLD (mp_size 1)

    @property
    def mp_rank(self) -> int:
        return self.rank % self.mp_size

    @property
    def dp_size(self) -> int:
        return self.world // self.mp_size

    @property
    def dp_rank(self) -> int:
        return self.rank // self.mp_size

    def mp_ranks(self) -> List[int]:
        first = self.dp_rank * self.mp_size
        return list(range(first, first + self.mp_size))

    def dp_ranks(self) -> List[int]:
        return list(range(self.mp_rank, self.world, self.mp_size))


def build_mesh(mp_size: Optional[int] = None) -> ParallelMesh:
    """Collective over WORLD: every rank creates every sub-group, in the same order."""
    if not (dist.is_available() and dist.is_initialized()):
        return ParallelMesh(world=1, rank=0, mp_size=1)
    world, rank = dist.get_world_size(), dist.get_rank()
    mp_size = world if not mp_size or mp_size <= 0 else int(mp_size)
    if world % mp_size:
        raise ValueError(f"world size {world} is not a multiple of the model-parallel size {mp_size}")
    mesh = ParallelMesh(world=world, rank=rank, mp_size=mp_size)
    if mp_size not in (1, world):
        for block in range(world // mp_size):
            ranks = list(range(block * mp_size, (block + 1) * mp_size))
            g = dist.new_group(ranks)
            if rank in ranks:
                mesh.mp_group = g
        for pos in range(mp_size):
            ranks = list(range(pos, world, mp_size))
            g = dist.new_group(ranks)
            if rank in ranks:
                mesh.dp_group = g
    return mesh


def model_parallel_size(parallel_mode: str, world: int, tp_size: int = 1, cp_size: int = 1, ep_size: int = 1,
                        pp_size: int = 1) -> int:
    """Ranks per model-parallel block for a training mode.  A size of 1 (the configuration default) next to a
    model-parallel mode means "the whole job"."""
    size = {"tp": tp_size, "cp": cp_size, "ep": ep_size, "pp": pp_size}.get(parallel_mode)
    if size is None:
        return 1
    return world if size <= 1 else min(int(size), world)


def data_parallel_size(parallel_mode: str, world: int, tp_size: int = 1, cp_size: int = 1, ep_size: int = 1,
                       pp_size: int = 1) -> int:
    """How many ranks draw different samples: the tensor-, context- or pipeline-parallel ranks of one block share their
    batch; every other mode (expert parallelism included) gives each rank a batch of its own."""
    if parallel_mode in ("tp", "cp", "pp"):
        return max(world // model_parallel_size(parallel_mode, world, tp_size, cp_size, ep_size, pp_size), 1)
    return world
