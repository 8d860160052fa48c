"""Resumable distributed sampler.

Semantics of ``astrai/dataset/sampler.py:8-93``: permutation from ``Generator(seed + epoch)``, wrap-around padding to
a multiple of the replica count (unless ``drop_last``), rank-strided slice, and a first epoch that skips
``start_iter % per_replica`` samples so a restarted run continues at the next unseen sample.
"""

from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist
from torch.utils.data import Sampler


class RDSampler(Sampler[int]):
    def __init__(self, data_source, start_epoch: int = 0, start_iter: int = 0, seed: int = 42, drop_last: bool = False,
                 shuffle: bool = True, process_group: Optional[dist.ProcessGroup] = None, partition=None):
        """``partition=(index, count)`` names this rank's share explicitly (ranks of one model-parallel block pass the
        same pair and so draw the same samples); otherwise the share follows the process group."""
        self.epoch, self.seed, self.drop_last, self.shuffle = start_epoch, seed, drop_last, shuffle
        self.num_samples = len(data_source)
        if partition is not None:
            self.rank, self.num_replicas = int(partition[0]), int(partition[1])
        elif process_group is not None:
            self.rank, self.num_replicas = dist.get_rank(process_group), dist.get_world_size(process_group)
        elif dist.is_available() and dist.is_initialized():
            self.rank, self.num_replicas = dist.get_rank(), dist.get_world_size()
        else:
            self.rank, self.num_replicas = 0, 1
        n, w = self.num_samples, self.num_replicas
        self.num_samples_per_replica = n // w if drop_last else -(-n // w)
        self.total_size = self.num_samples_per_replica * w
        self.iter = start_iter % self.num_samples_per_replica if self.num_samples_per_replica else 0
        self._pending = None

    def _plan(self):
        if self.shuffle:
            g = torch.Generator()
            g.manual_seed(self.seed + self.epoch)
            order = torch.randperm(self.num_samples, generator=g).tolist()
        else:
            order = list(range(self.num_samples))
        if not self.drop_last and order and len(order) < self.total_size:
            missing = self.total_size - len(order)  # wrap around, more than once when there are fewer samples than ranks
            order += (order * (-(-missing // len(order))))[:missing]
        mine = order[self.rank:self.total_size:self.num_replicas]
        self._pending = mine[self.iter:]

    def __iter__(self):
        if self._pending is None:
            self._plan()
        for idx in self._pending:
            self.iter += 1
            yield idx
        self.epoch += 1
        self._pending = None
        self.iter %= max(self.num_samples_per_replica, 1)

    def __len__(self):
        return max(self.num_samples_per_replica - self.iter, 0)
