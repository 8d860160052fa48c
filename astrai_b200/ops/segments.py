"""Causal attention restricted to runs of tokens, described by boundaries instead of a dense boolean mask.

The reference builds ``[B, 1, S, S]`` boolean masks for its masked objectives - same-document-and-causal for packed SFT
batches (``astrai/trainer/strategy.py:87-100``), key-is-not-padding-and-causal for DPO / GRPO (``:422-474``,
``:546-642``) - which costs O(S^2) memory and forces the library's non-flash attention.  Both masks have the same shape:
every row of the batch is a sequence of *runs* (documents; or left padding, real tokens, right padding) and a token
attends causally inside its own run.  :class:`AttentionSegments` records the runs as cumulative boundaries over the
flattened ``[B*S]`` token axis, which is exactly the ``cu_seqlens`` input of the variable-length flash kernels; the dense
mask is still available (:meth:`to_dense`) for the CPU path and for back ends without a variable-length kernel.

Rows of padding form runs of their own: their outputs differ from the dense-mask result (a padding query sees the
padding before it instead of nothing) and are never read, because the loss masks them out.

Boundaries are computed on the host from tensors that are still on the host when a batch arrives from the data loader,
so no device synchronisation is involved.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch
from torch import Tensor


@dataclass
class AttentionSegments:
    bounds: List[int]          # cumulative run boundaries over the flattened [B*S] axis, starting at 0, ending at B*S
    batch: int
    seq_len: int
    rows: Optional[List[List[int]]] = None  # per batch row: run boundaries inside the row (kept for drop_last)
    _cu: Optional[Tensor] = None

    @property
    def n_runs(self) -> int:
        return len(self.bounds) - 1

    @property
    def max_len(self) -> int:
        return max((b - a for a, b in zip(self.bounds[:-1], self.bounds[1:])), default=0)

    def cu_seqlens(self, device) -> Tensor:
        if self._cu is None or self._cu.device != torch.device(device):
            self._cu = torch.tensor(self.bounds, dtype=torch.int32).to(device, non_blocking=True)
        return self._cu

    def drop_last(self) -> "AttentionSegments":
        """The same runs for rows shortened by their last token (inputs of a next-token objective)."""
        rows = []
        for r in self.rows:
            cut = [min(b, self.seq_len - 1) for b in r]
            rows.append(sorted(set(cut)))
        return from_row_bounds(rows, self.seq_len - 1)

    def to_dense(self, device=None) -> Tensor:
        """``[B, 1, S, S]`` bool, True = attend: same run and causal."""
        total = self.batch * self.seq_len
        run_id = torch.zeros(total, dtype=torch.long)
        for i, (a, b) in enumerate(zip(self.bounds[:-1], self.bounds[1:])):
            run_id[a:b] = i
        run_id = run_id.view(self.batch, self.seq_len)
        same = run_id[:, :, None] == run_id[:, None, :]
        causal = torch.ones(self.seq_len, self.seq_len, dtype=torch.bool).tril()
        out = (same & causal)[:, None]
        return out.to(device) if device is not None else out


def from_row_bounds(rows: List[List[int]], seq_len: int) -> AttentionSegments:
    """``rows[b]`` lists the run boundaries inside row ``b`` (0 and ``seq_len`` are added when missing)."""
    bounds = [0]
    norm = []
    for b, r in enumerate(rows):
        inner = sorted({0, seq_len, *[x for x in r if 0 < x < seq_len]})
        norm.append(inner)
        bounds.extend(b * seq_len + x for x in inner[1:])
    return AttentionSegments(bounds=bounds, batch=len(rows), seq_len=seq_len, rows=norm)


def from_position_ids(position_ids: Tensor) -> AttentionSegments:
    """Packed documents: a new document starts wherever the position does not grow (reference rule)."""
    pos = position_ids.detach().cpu()
    b, s = pos.shape
    starts = (pos[:, 1:] <= pos[:, :-1])
    rows = [(starts[i].nonzero().flatten() + 1).tolist() for i in range(b)]
    return from_row_bounds(rows, s)


def from_valid_mask(valid: Tensor) -> Optional[AttentionSegments]:
    """Key padding: ``valid [B, S]`` marks real tokens.  Returns ``None`` when the real tokens of some row are not one
    contiguous run (padding in the middle), which the run form cannot express."""
    v = valid.detach().cpu().bool()
    b, s = v.shape
    rows = []
    for i in range(b):
        idx = v[i].nonzero().flatten()
        if idx.numel() == 0:
            rows.append([])
            continue
        first, last = int(idx[0]), int(idx[-1])
        if idx.numel() != last - first + 1:
            return None
        rows.append([first, last + 1])
    return from_row_bounds(rows, s)
