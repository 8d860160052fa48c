"""Tensor-parallel serving: one model replica cut over the ranks of a group, every rank running the same scheduler.

The reference serves on one GPU (``astrai/inference/network/app.py:108-130`` builds one engine on one device).  Here a
decoder is cut Megatron-style for inference - attention heads and FFN columns divided over ``tp`` ranks, embedding, norms
and the output projection replicated - and the partial outputs of every attention and FFN block are summed with ONE
all-reduce each (the sequence-sharded all-gather / reduce-scatter form used for training needs row blocks of 256 tokens
and does not fit decode steps of a few rows).  Each rank keeps the K / V of its own heads only, so the paged pool shrinks
by ``tp`` per GPU.

Scheduling is SPMD: every rank runs the *same* :class:`~astrai_b200.inference.scheduler.InferenceScheduler` loop on the
same queue contents, so page allocation, batching and admission decisions are identical everywhere without being
communicated.  Two things are communicated per loop iteration, both from the first rank of the group
(:class:`ReplicatedControl`): the requests that arrived (or were cancelled) since the last iteration, as one object
broadcast, and the sampled tokens of the step (so that one random stream decides for all).  Streaming callbacks fire
on the first rank only, which is where the HTTP front end runs; the other ranks call ``scheduler.follow()``.
"""

from __future__ import annotations

import logging
from typing import Any, Dict, List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn
from torch import Tensor

logger = logging.getLogger(__name__)


def _rows(linear: nn.Module, lo: int, hi: int):
    linear.weight.data = linear.weight.data[lo:hi].contiguous()
    if getattr(linear, "bias", None) is not None:
        linear.bias.data = linear.bias.data[lo:hi].contiguous()
    linear.out_dim = hi - lo


def _cols(linear: nn.Module, lo: int, hi: int, keep_bias: bool):
    linear.weight.data = linear.weight.data[:, lo:hi].contiguous()
    if getattr(linear, "bias", None) is not None and not keep_bias:
        linear.bias.data = torch.zeros_like(linear.bias.data)  # the bias is added once: by the rank that keeps it
    linear.in_dim = hi - lo


def _shard_attention(mod, tp: int, rank: int):
    hq, hkv, d = mod.n_heads, mod.n_kv_heads, mod.head_dim
    if hkv % tp or hq % tp:
        raise ValueError(f"{hq} query / {hkv} key-value heads do not divide over {tp} tensor-parallel ranks")
    q, kv = hq // tp * d, hkv // tp * d
    _rows(mod.q_proj, rank * q, (rank + 1) * q)
    _rows(mod.k_proj, rank * kv, (rank + 1) * kv)
    _rows(mod.v_proj, rank * kv, (rank + 1) * kv)
    if getattr(mod, "use_gated_attention", False):
        _rows(mod.gate, rank * q, (rank + 1) * q)
    _cols(mod.o_proj, rank * q, (rank + 1) * q, keep_bias=rank == 0)
    mod.n_heads, mod.n_kv_heads = hq // tp, hkv // tp
    mod.fused_qkv = None


def _shard_mlp(mod, tp: int, rank: int):
    f = mod.gate.weight.shape[0]
    if f % tp:
        raise ValueError(f"an FFN width of {f} does not divide over {tp} tensor-parallel ranks")
    lo, hi = rank * (f // tp), (rank + 1) * (f // tp)
    _rows(mod.gate, lo, hi)
    _rows(mod.up, lo, hi)
    _cols(mod.down, lo, hi, keep_bias=rank == 0)
    mod.fused_gate_up = None


def shard_for_inference_(model: nn.Module, tp: int, rank: int, group=None) -> nn.Module:
    """Cut ``model`` (every rank holds the same full weights on entry) down to this rank's share, in place, and make the
    attention and FFN blocks sum their partial outputs over ``group``.  For inference only: the cut tensors carry no
    gradient bookkeeping and the state dict no longer has the checkpoint's shapes."""
    from astrai_b200.models.attention import GQA
    from astrai_b200.models.ffn import MLP, DeepSeekMoE

    if tp <= 1:
        return model

    def summed(tensor: Tensor) -> Tensor:
        dist.all_reduce(tensor, group=group)
        return tensor

    def attention_hook(_mod, _args, out):
        return summed(out.contiguous())

    def ffn_hook(_mod, _args, out):
        out["hidden_states"] = summed(out["hidden_states"].contiguous())
        return out

    with torch.no_grad():
        for layer in model.layers:
            attn, ffn = layer.attention, layer.mlp
            if not isinstance(attn, GQA):
                raise NotImplementedError(f"tensor-parallel serving cuts grouped-query attention; got {type(attn).__name__}")
            _shard_attention(attn, tp, rank)
            attn.register_forward_hook(attention_hook)
            if isinstance(ffn, MLP):
                _shard_mlp(ffn, tp, rank)
            elif isinstance(ffn, DeepSeekMoE):  # the router stays whole; every expert is cut like a dense FFN
                for expert in list(ffn.routed_experts) + list(ffn.shared_experts):
                    _shard_mlp(expert, tp, rank)
                ffn.stacked_experts = None
            else:
                raise NotImplementedError(f"tensor-parallel serving does not know the FFN {type(ffn).__name__}")
            ffn.register_forward_hook(ffn_hook)
    model.tp_size, model.tp_rank = tp, rank
    model.local_config = LocalHeads(model.config, tp)
    return model


class LocalHeads:
    """The model configuration as one tensor-parallel rank sees it where cache and workspace sizes are derived: its own
    share of the heads, the same head dimension.  Everything else reads through to the real configuration."""

    def __init__(self, config, tp: int):
        self._config, self._tp = config, tp

    def __getattr__(self, name: str):
        value = getattr(self._config, name)
        if name in ("num_attention_heads", "num_key_value_heads", "hidden_size") and value is not None:
            return value // self._tp  # hidden_size // num_attention_heads (the head dimension) stays what it was
        return value


class ReplicatedControl:
    """What the ranks of one serving replica tell each other, always from the group's first rank."""

    def __init__(self, group=None):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.src = dist.get_global_rank(group, 0) if group is not None else 0
        self.leader = self.rank == 0
        # object broadcasts of request lists go through a CPU (gloo) group when the data group is NCCL
        self._cpu_group = group
        if dist.get_backend(group) == "nccl":
            ranks = dist.get_process_group_ranks(group) if group is not None else list(range(dist.get_world_size()))
            self._cpu_group = dist.new_group(ranks, backend="gloo")

    def share(self, payload: Optional[Dict[str, Any]]) -> Dict[str, Any]:
        """The leader's ``payload`` on every rank (followers pass ``None``)."""
        box = [payload if self.leader else None]
        dist.broadcast_object_list(box, src=self.src, group=self._cpu_group)
        return box[0]

    def share_tokens(self, *tensors: Tensor):
        """Overwrite the followers' sampled tokens (and log-probabilities) with the leader's."""
        for t in tensors:
            dist.broadcast(t, src=self.src, group=self.group)
