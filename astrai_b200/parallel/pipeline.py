"""Pipeline parallelism for :class:`AutoRegressiveLM`: contiguous layer ranges per stage, 1F1B micro-batch schedule.

Stage ``s`` of ``P`` owns decoder layers ``[bounds[s], bounds[s+1])``; the first stage also owns the token embedding, the
last one the final norm, the output projection and the loss.  One optimizer step runs ``M`` micro-batches through the
non-interleaved one-forward-one-backward schedule: stage ``s`` does ``min(P - 1 - s, M)`` warm-up forwards, then
alternates forward / backward, then drains its remaining backwards, so at most ``P - s`` micro-batches of activations are
alive on a stage.  Activations travel forward and their gradients backward as point-to-point messages of the process
group (NCCL over NVLink between GPUs of a node, Gloo in the CPU tests); every rank of a stage pair posts its send and
receive of one schedule slot together (``batch_isend_irecv``), which keeps the neighbours from blocking each other.

Gradients accumulate in the stage's parameters over the micro-batches (the loss of each micro-batch is divided by ``M``),
exactly like gradient accumulation on one device; the optimizer step is the caller's, per stage.  A tied output
projection is not supported across stages (the embedding and the head live on different ranks).

The reference has no pipeline parallelism: its parallel modes are none / DDP / FSDP
(``astrai/config/train_config.py:15``; ``astrai/parallel/executor.py:254-428``).
"""

from __future__ import annotations

from typing import Callable, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist
from torch import Tensor, nn


def split_layers(n_layers: int, n_stages: int) -> List[int]:
    """Layer boundaries ``[b_0 = 0, ..., b_P = n_layers]``: as even as possible, the earlier stages take the remainder
    (the last stage also carries the head and the loss)."""
    if not 1 <= n_stages <= n_layers:
        raise ValueError(f"cannot cut {n_layers} layers into {n_stages} stages")
    base, extra = divmod(n_layers, n_stages)
    bounds = [0]
    for s in range(n_stages):
        bounds.append(bounds[-1] + base + (1 if s < extra else 0))
    return bounds


def schedule_1f1b(n_stages: int, stage: int, n_micro: int) -> List[Tuple[str, int]]:
    """The order of this stage's steps: ``("F", i)`` / ``("B", i)`` for micro-batch ``i``."""
    warm = min(n_stages - 1 - stage, n_micro)
    steps: List[Tuple[str, int]] = [("F", i) for i in range(warm)]
    f, b = warm, 0
    while f < n_micro:
        steps.append(("F", f))
        steps.append(("B", b))
        f, b = f + 1, b + 1
    while b < n_micro:
        steps.append(("B", b))
        b += 1
    return steps


class PipelineStage(nn.Module):
    """The part of an :class:`AutoRegressiveLM` that one stage runs.  Parameters are shared with (not copied from) the
    model it was cut from, so checkpoints keep the reference's key names: a stage saves / loads its own keys."""

    def __init__(self, model: nn.Module, n_stages: int, stage: int, bounds: Optional[Sequence[int]] = None):
        super().__init__()
        if getattr(model, "tied", False) and n_stages > 1:
            raise ValueError("pipeline parallelism needs an untied output projection (tie_word_embeddings=False)")
        self.n_stages, self.stage = n_stages, stage
        self.bounds = list(bounds) if bounds is not None else split_layers(len(model.layers), n_stages)
        self.first, self.last = stage == 0, stage == n_stages - 1
        self.rotary_embedding = model.rotary_embedding
        self.embed_tokens = model.embed_tokens if self.first else None
        self.layers = nn.ModuleList(model.layers[self.bounds[stage]:self.bounds[stage + 1]])
        self.norm = model.norm if self.last else None
        self.lm_head = model.lm_head if self.last else None
        self.hidden_size = model.config.hidden_size
        # the whole model reports the MEAN of its layers' router losses: every stage contributes its layers' share of it
        n_routed = sum(1 for layer in model.layers if hasattr(getattr(layer, "mlp", None), "router"))
        self.aux_scale = 1.0 / max(n_routed, 1)

    def owned_keys(self, model: nn.Module) -> List[str]:
        """State-dict keys of the full model that live on this stage."""
        mine = {id(p) for p in self.parameters()}
        return [k for k, v in model.state_dict(keep_vars=True).items() if id(v) in mine]

    def forward(self, x: Tensor, position_ids: Optional[Tensor] = None, attention=None):
        """First stage: ``x`` are token ids ``[B, S]``; later stages: hidden states ``[B, S, H]``.  ``attention`` is what
        the whole model takes as ``input_mask`` (a padding / dense mask or the run boundaries of packed documents);
        without it attention is causal.  Returns hidden states, or logits on the last stage, plus this stage's share of
        the model's router auxiliary loss (its layers' losses over the model's number of routed layers; ``None`` if it
        has none): summed over the stages that is the mean the whole model reports."""
        from astrai_b200.models.lm import expand_mask

        if self.first:
            x = self.embed_tokens(x)
        rotary = self.rotary_embedding(x, position_ids)
        mask = expand_mask(attention)
        aux = None
        for layer in self.layers:
            out = layer(x, rotary, mask, None, mask is None, None)
            x = out["hidden_states"]
            if out.get("aux_loss") is not None:
                aux = out["aux_loss"] if aux is None else aux + out["aux_loss"]
        if self.last:
            x = self.lm_head(self.norm(x))
        return x, (aux * self.aux_scale if aux is not None else None)


def _default_loss(logits: Tensor, targets: Tensor) -> Tensor:
    return torch.nn.functional.cross_entropy(logits.reshape(-1, logits.size(-1)).float(), targets.reshape(-1))


class PipelineParallel:
    """Runs optimizer steps of a model cut into stages over the ranks of ``group`` (rank ``r`` of the group is stage ``r``)."""

    def __init__(self, model: nn.Module, group=None, bounds: Optional[Sequence[int]] = None,
                 loss_fn: Callable[[Tensor, Tensor], Tensor] = _default_loss, aux_loss_coef: float = 0.0):
        self.group = group
        self.n_stages = dist.get_world_size(group)
        self.stage_index = dist.get_rank(group)
        self.stage = PipelineStage(model, self.n_stages, self.stage_index, bounds)
        self.loss_fn, self.aux_loss_coef = loss_fn, aux_loss_coef
        self._prev = None if self.stage.first else dist.get_global_rank(group, self.stage_index - 1) if group is not None else self.stage_index - 1
        self._next = None if self.stage.last else dist.get_global_rank(group, self.stage_index + 1) if group is not None else self.stage_index + 1

    def parameters(self):
        return self.stage.parameters()

    # -- point-to-point helpers: everything of one schedule slot is posted together ------------------------------------
    def _exchange(self, sends: List[Tuple[Tensor, int]], recvs: List[Tuple[Tensor, int]]):
        ops = [dist.P2POp(dist.isend, t.contiguous(), peer, self.group) for t, peer in sends]
        ops += [dist.P2POp(dist.irecv, t, peer, self.group) for t, peer in recvs]
        if ops:
            for work in dist.batch_isend_irecv(ops):
                work.wait()

    def train_step(self, input_ids: Optional[Tensor], targets: Optional[Tensor], n_micro: int,
                   micro_shape: Optional[Tuple[int, int]] = None, dtype: Optional[torch.dtype] = None,
                   loss_scale: float = 1.0, micro_kwargs: Optional[Sequence[dict]] = None,
                   weights: Optional[Sequence[float]] = None, loss_fn: Optional[Callable] = None) -> Optional[Tensor]:
        """One accumulation window (gradients are those of ``loss_scale`` times the window's loss).  ``input_ids``
        ``[B, S]`` is needed on the first stage, ``targets`` ``[B, S]`` on the last; ``B`` must be a multiple of
        ``n_micro``.  Stages in the middle pass ``micro_shape = (B / n_micro, S)``.

        ``micro_kwargs[i]`` are keyword arguments of the stage's forward for piece ``i`` (``position_ids``,
        ``attention``), the same on every stage.  ``weights[i]`` is the share of piece ``i`` in the window's loss
        (default ``1 / n_micro`` each: the mean of the pieces' means); an objective that averages over a varying number
        of tokens per piece passes that piece's share of the tokens, which makes the window's loss the mean over all
        its tokens.  ``targets`` may also be a list with one object per piece and ``loss_fn(logits, object)`` the objective
        of this window (sequence-level losses carry ids, masks and reference values per piece).  Returns the window's
        loss on the last stage, ``None`` elsewhere.  Gradients are left in ``.grad``."""
        st = self.stage
        if weights is None:
            weights = [1.0 / n_micro] * n_micro
        if micro_kwargs is None:
            micro_kwargs = [{}] * n_micro
        if len(weights) != n_micro or len(micro_kwargs) != n_micro:
            raise ValueError(f"{n_micro} pieces need {n_micro} weights and keyword sets")
        dev = next(st.parameters()).device
        dtype = dtype or next(st.parameters()).dtype
        if st.first:
            micro_in = input_ids.chunk(n_micro, dim=0)
            micro_shape = tuple(micro_in[0].shape)
        loss_fn = loss_fn or self.loss_fn
        if st.last and targets is not None:
            micro_tg = list(targets) if isinstance(targets, (list, tuple)) else targets.chunk(n_micro, dim=0)
            if micro_shape is None:
                micro_shape = tuple(micro_tg[0].shape)
        if micro_shape is None:
            raise ValueError("a middle stage needs micro_shape")
        act_shape = (micro_shape[0], micro_shape[1], st.hidden_size)
        losses: List[Tensor] = []
        live: List[Tuple[Tensor, Tensor]] = []  # (input, output) of the forwards whose backward is still to come

        def new_act():
            return torch.empty(act_shape, dtype=dtype, device=dev)

        def recv_forward(i):
            if st.first:
                return micro_in[i]
            x = new_act()
            self._exchange([], [(x, self._prev)])
            return x.requires_grad_(True)

        def forward(i, x):
            y, aux = st(x, **micro_kwargs[i])
            if st.last:
                loss = loss_fn(y, micro_tg[i])
                losses.append(loss.detach() * weights[i])
                y = loss * (loss_scale * weights[i])
                if aux is not None and self.aux_loss_coef:  # the auxiliary loss is a plain mean over the pieces
                    y = y + aux * (self.aux_loss_coef * loss_scale / n_micro)
            elif aux is not None and self.aux_loss_coef:  # the stage's own share of the auxiliary loss
                (self.aux_loss_coef * aux * (loss_scale / n_micro)).backward(retain_graph=True)
            live.append((x, y))
            return y

        def backward(gy):
            x, y = live.pop(0)
            if st.last:
                y.backward()
            else:
                y.backward(gy)
            return None if st.first else x.grad

        # A send towards one neighbour and the receive from the same neighbour that follows it in the schedule are posted
        # as ONE batch: posted one after the other, two neighbours that both send first would wait for each other.
        warm = min(self.n_stages - 1 - self.stage_index, n_micro)
        steady = n_micro - warm
        for i in range(warm):
            y = forward(i, recv_forward(i))
            if not st.last:
                self._exchange([(y.detach(), self._next)], [])
        x = recv_forward(warm) if steady > 0 else None
        for k in range(steady):
            y = forward(warm + k, x)
            gy = None
            if not st.last:
                gy = new_act()
                self._exchange([(y.detach(), self._next)], [(gy, self._next)])
            gx = backward(gy)
            more = k + 1 < steady
            if st.first:
                x = micro_in[warm + k + 1] if more else None
            elif more:
                x = new_act()
                self._exchange([(gx, self._prev)], [(x, self._prev)])
                x.requires_grad_(True)
            else:
                self._exchange([(gx, self._prev)], [])
        for _ in range(warm):
            gy = None
            if not st.last:
                gy = new_act()
                self._exchange([], [(gy, self._next)])
            gx = backward(gy)
            if not st.first:
                self._exchange([(gx, self._prev)], [])
        return torch.stack(losses).sum() if st.last else None

    @torch.no_grad()
    def forward_only(self, input_ids: Optional[Tensor], micro_shape: Optional[Tuple[int, int]] = None,
                     dtype: Optional[torch.dtype] = None, **stage_kwargs) -> Optional[Tensor]:
        """Evaluation pass of one batch through the stages; logits on the last stage, ``None`` elsewhere.
        ``stage_kwargs`` (``position_ids``, ``attention``) go to every stage's forward."""
        st = self.stage
        dev = next(st.parameters()).device
        dtype = dtype or next(st.parameters()).dtype
        if st.first:
            x = input_ids
        else:
            x = torch.empty((micro_shape[0], micro_shape[1], st.hidden_size), dtype=dtype, device=dev)
            self._exchange([], [(x, self._prev)])
        y, _ = st(x, **stage_kwargs)
        if st.last:
            return y
        self._exchange([(y, self._next)], [])
        return None
