"""Matrix-aware optimizers and their AdamW companions.

* ``Muon``: momentum -> Newton-Schulz orthogonalisation (5 quintic iterations, bf16 GEMMs on the tcgen05 kernel when
  the matrix lives on a GPU) -> decoupled weight decay, as ``torch.optim.Muon`` does in the reference
  (``astrai/optim/muon_adamw.py:60-68``).
* ``Nora``: row-wise tangent projection + row normalisation with a Nesterov EMA, LR scaled by
  ``sqrt(max(1, d_out / d_in))`` (``astrai/optim/nora_nadamw.py:27-136``).
* ``Mano``: tangent projection alternating between the two matrix axes, LR x ``0.2 * sqrt(dim)``
  (``astrai/optim/mano_adamw.py:26-117``).
* ``NAdamW``: AdamW with the Nesterov first-moment estimate (``nora_nadamw.py:139-217``).
* ``partition_optimizer_parameters``: which tensors go to the matrix optimizer (2-D weights of internal ``Linear``
  layers), which get weight decay, which do not (embeddings, norms, biases, ``lm_head``, LoRA factors).
Composite front ends ``muon_adamw``, ``nora_nadamw``, ``mano_adamw`` take the MODEL, like the reference.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, List

import torch
from torch import Tensor, nn
from torch.optim import Optimizer

from astrai_b200.optim.base import CompositeOptimizer, OptimizerFactory, UntracedOptimizer
from astrai_b200.optim.fused_adamw import FusedAdamW

NORA_EPS = 1e-10


def _check(cond: bool, msg: str):
    if not cond:
        raise ValueError(msg)


def _grad_of(p: Tensor):
    return p.grad


# ------------------------------------------------------------------------------------------------- Muon
NS_COEFFS = (3.4445, -4.7750, 2.0315)


def _mm(a: Tensor, b_t: Tensor) -> Tensor:
    """a @ b_t.T with the tcgen05 kernel for bf16 CUDA operands."""
    if a.is_cuda and a.dtype == torch.bfloat16:
        from astrai_b200 import ops

        return ops.gemm(a.contiguous(), b_t.contiguous())
    return a @ b_t.t()


def newton_schulz(grad: Tensor, steps: int = 5, eps: float = 1e-7) -> Tensor:
    """Approximate the orthogonal polar factor of a matrix with the quintic Newton-Schulz iteration."""
    a, b, c = NS_COEFFS
    x = grad.to(torch.bfloat16)
    tall = x.size(0) > x.size(1)
    if tall:
        x = x.t().contiguous()
    x = x / (x.norm() + eps)
    for _ in range(steps):
        gram = _mm(x, x)                                  # X X^T
        poly = b * gram + c * _mm(gram, gram)             # gram is symmetric: gram @ gram == gram @ gram.T
        x = a * x + _mm(poly, x.t().contiguous())         # poly @ X
    return (x.t() if tall else x).to(grad.dtype)


def muon_lr(lr: float, shape, mode: str) -> float:
    rows, cols = shape[-2], shape[-1]
    if mode == "match_rms_adamw":
        return lr * 0.2 * math.sqrt(max(rows, cols))
    return lr * math.sqrt(max(1.0, rows / cols))


class Muon(UntracedOptimizer):
    def __init__(self, params, lr: float = 1e-3, weight_decay: float = 0.1, momentum: float = 0.95, nesterov: bool = True,
                 ns_steps: int = 5, adjust_lr_fn: str = "original", eps: float = 1e-7):
        _check(lr >= 0, f"Invalid learning rate: {lr}")
        _check(adjust_lr_fn in ("original", "match_rms_adamw"), f"Invalid adjust_lr_fn: {adjust_lr_fn}")
        super().__init__(params, dict(lr=lr, weight_decay=weight_decay, momentum=momentum, nesterov=nesterov,
                                      ns_steps=ns_steps, adjust_lr_fn=adjust_lr_fn, eps=eps))
        for g in self.param_groups:
            for p in g["params"]:
                _check(p.ndim == 2, f"Muon only supports 2D matrices, got shape {tuple(p.shape)}")

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for g in self.param_groups:
            for p in g["params"]:
                grad = _grad_of(p)
                if grad is None:
                    continue
                st = self.state[p]
                buf = st.get("momentum_buffer")
                if buf is None:
                    buf = st["momentum_buffer"] = torch.zeros_like(grad)
                buf.lerp_(grad, 1 - g["momentum"])
                update = grad.lerp(buf, g["momentum"]) if g["nesterov"] else buf
                direction = newton_schulz(update, g["ns_steps"], g["eps"])
                if g["weight_decay"]:
                    p.mul_(1 - g["lr"] * g["weight_decay"])
                p.add_(direction.to(p.dtype), alpha=-muon_lr(g["lr"], p.shape, g["adjust_lr_fn"]))
        return loss


# ------------------------------------------------------------------------------------------------- Nora
def _unit_rows(t: Tensor, eps: float) -> Tensor:
    return t / t.norm(dim=-1, keepdim=True).clamp(min=eps)


def nora_direction(update: Tensor, param: Tensor, eps: float = NORA_EPS) -> Tensor:
    """Remove from each row of ``update`` its component along the matching parameter row, then normalise the row."""
    theta = _unit_rows(param.float(), eps)
    u = update.float()
    return _unit_rows(u - (u * theta).sum(-1, keepdim=True) * theta, eps).to(update.dtype)


def nora_lr_scale(lr: float, shape) -> float:
    return lr * math.sqrt(max(1.0, shape[-2] / shape[-1]))


def _require_whole_rows(p: Tensor):
    try:
        from torch.distributed.tensor import DTensor, Shard
    except Exception:  # noqa: BLE001
        return
    if isinstance(p, DTensor):
        for pl in p.placements:
            if isinstance(pl, Shard) and pl.dim % p.ndim == p.ndim - 1:
                raise ValueError("Nora requires complete parameter rows, but this DTensor is sharded along its last dimension")


class Nora(UntracedOptimizer):
    def __init__(self, params, lr: float = 5e-3, weight_decay: float = 0.0, momentum: float = 0.95, beta: float = 0.95,
                 nesterov: bool = True, eps: float = NORA_EPS):
        _check(lr >= 0, f"Invalid learning rate: {lr}")
        _check(weight_decay >= 0, f"Invalid weight decay: {weight_decay}")
        _check(0 <= momentum <= 1, f"Invalid momentum: {momentum}")
        _check(0 <= beta < 1, f"Invalid beta: {beta}")
        _check(eps > 0, f"Invalid epsilon: {eps}")
        super().__init__(params, dict(lr=lr, weight_decay=weight_decay, momentum=momentum, beta=beta, nesterov=nesterov, eps=eps))
        for g in self.param_groups:
            for p in g["params"]:
                _check(p.ndim == 2, f"Nora only supports 2D matrices, got shape {tuple(p.shape)}")
                _require_whole_rows(p)

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for g in self.param_groups:
            for p in g["params"]:
                grad = _grad_of(p)
                if grad is None:
                    continue
                if grad.is_sparse:
                    raise RuntimeError("Nora does not support sparse gradients")
                st = self.state[p]
                buf = st.get("momentum_buffer")
                if buf is None:
                    buf = st["momentum_buffer"] = torch.zeros_like(grad)
                buf.lerp_(grad, 1 - g["beta"])
                update = grad.lerp(buf, g["momentum"]) if g["nesterov"] else buf
                direction = nora_direction(update, p, g["eps"])
                if g["weight_decay"]:
                    p.mul_(1 - g["lr"] * g["weight_decay"])
                p.add_(direction, alpha=-nora_lr_scale(g["lr"], p.shape))
        return loss


# ------------------------------------------------------------------------------------------------- Mano
class Mano(UntracedOptimizer):
    def __init__(self, params, lr: float = 1e-3, weight_decay: float = 0.1, momentum: float = 0.95, nesterov: bool = True,
                 eps: float = 1e-8):
        _check(lr >= 0, f"Invalid learning rate: {lr}")
        _check(weight_decay >= 0, f"Invalid weight decay: {weight_decay}")
        _check(0 <= momentum <= 1, f"Invalid momentum: {momentum}")
        _check(eps > 0, f"Invalid epsilon: {eps}")
        super().__init__(params, dict(lr=lr, weight_decay=weight_decay, momentum=momentum, nesterov=nesterov, eps=eps, steps=0))
        for g in self.param_groups:
            for p in g["params"]:
                _check(p.ndim == 2, f"Mano only supports 2D matrices, got shape {tuple(p.shape)}")

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for g in self.param_groups:
            axis = int(g["steps"] % 2)  # alternate between columns and rows
            for p in g["params"]:
                grad = _grad_of(p)
                if grad is None:
                    continue
                if grad.is_sparse:
                    raise RuntimeError("Mano does not support sparse gradients")
                st = self.state[p]
                buf = st.get("momentum_buffer")
                if buf is None:
                    buf = st["momentum_buffer"] = torch.zeros_like(grad)
                buf.mul_(g["momentum"]).add_(grad)
                update = grad.add(buf, alpha=g["momentum"]) if g["nesterov"] else buf
                tangent = update - (update * p).sum(dim=axis, keepdim=True) * p
                direction = tangent / (tangent.norm(p=2, dim=axis, keepdim=True) + g["eps"])
                if g["weight_decay"]:
                    p.mul_(1 - g["lr"] * g["weight_decay"])
                p.add_(direction, alpha=-g["lr"] * 0.2 * math.sqrt(direction.shape[axis]))
            g["steps"] += 1
        return loss


# ------------------------------------------------------------------------------------------------- NAdamW
class NAdamW(UntracedOptimizer):
    def __init__(self, params, lr: float = 3e-4, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.1):
        _check(lr >= 0, f"Invalid learning rate: {lr}")
        _check(0 <= betas[0] < 1 and 0 <= betas[1] < 1, f"Invalid betas: {betas}")
        _check(eps > 0, f"Invalid epsilon: {eps}")
        _check(weight_decay >= 0, f"Invalid weight decay: {weight_decay}")
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay))

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for g in self.param_groups:
            b1, b2 = g["betas"]
            for p in g["params"]:
                grad = _grad_of(p)
                if grad is None:
                    continue
                if grad.is_sparse:
                    raise RuntimeError("NAdamW does not support sparse gradients")
                st = self.state[p]
                if not st:
                    st["step"], st["m"], st["v"] = 0, torch.zeros_like(p), torch.zeros_like(p)
                st["step"] += 1
                m, v = st["m"], st["v"]
                m.mul_(b1).add_(grad, alpha=1 - b1)
                v.mul_(b2).addcmul_(grad, grad, value=1 - b2)
                look_ahead = (b1 * m + (1 - b1) * grad) / (1 - b1 ** st["step"])
                denom = (v / (1 - b2 ** st["step"])).sqrt().add_(g["eps"])
                if g["weight_decay"]:
                    p.mul_(1 - g["lr"] * g["weight_decay"])
                p.addcdiv_(look_ahead, denom, value=-g["lr"])
        return loss


# ------------------------------------------------------------------------------------------------- partition + composites
@dataclass
class OptimizerParameterGroups:
    nora: List[Tensor]
    nadamw_decay: List[Tensor]
    nadamw_no_decay: List[Tensor]


def partition_optimizer_parameters(model: nn.Module) -> OptimizerParameterGroups:
    from astrai_b200.models.layers import Embedding, Linear, RMSNorm
    from astrai_b200.models.lora import LoRALinear

    matrix_ids, plain_ids = set(), set()
    for name, mod in model.named_modules():
        if isinstance(mod, (LoRALinear, Embedding, RMSNorm)):
            plain_ids.update(id(p) for p in mod.parameters(recurse=False) if p.requires_grad)
        elif isinstance(mod, Linear):
            if mod.bias is not None and mod.bias.requires_grad:
                plain_ids.add(id(mod.bias))
            if mod.weight.requires_grad:
                if name.rsplit(".", 1)[-1] == "lm_head":
                    plain_ids.add(id(mod.weight))
                elif mod.weight.ndim == 2:
                    matrix_ids.add(id(mod.weight))
    groups = OptimizerParameterGroups([], [], [])
    seen = set()
    for p in model.parameters():
        if not p.requires_grad or id(p) in seen:
            continue
        seen.add(id(p))
        if id(p) in plain_ids or p.ndim <= 1:
            groups.nadamw_no_decay.append(p)
        elif id(p) in matrix_ids:
            groups.nora.append(p)
        else:
            groups.nadamw_decay.append(p)
    return groups


def _all_params(g: OptimizerParameterGroups) -> List[Tensor]:
    params = [*g.nora, *g.nadamw_decay, *g.nadamw_no_decay]
    if not params:
        raise ValueError("Cannot build an optimizer for a model with no trainable parameters")
    return params


def _decay_groups(g: OptimizerParameterGroups, weight_decay: float):
    out = []
    if g.nadamw_decay:
        out.append({"params": g.nadamw_decay, "weight_decay": weight_decay})
    if g.nadamw_no_decay:
        out.append({"params": g.nadamw_no_decay, "weight_decay": 0.0})
    return out


@OptimizerFactory.register("muon_adamw")
class MuonAdamW(CompositeOptimizer):
    """Muon on matrices that are not norms / biases / embeddings / ``lm_head`` (selected by NAME, as the reference does);
    AdamW(betas 0.9, 0.95, no weight decay) on everything else."""

    optimizer_name = "muon_adamw"

    def __init__(self, model: nn.Module, lr: float = 3e-4, weight_decay: float = 0.1, momentum: float = 0.95,
                 nesterov: bool = True, ns_steps: int = 5, adjust_lr_fn: str = "match_rms_adamw"):
        matrices, others, seen = [], [], set()
        for name, p in model.named_parameters():
            if not p.requires_grad or id(p) in seen:
                continue
            seen.add(id(p))
            skip = any(tag in name for tag in ("norm", "bias", "embed", "lm_head"))
            (matrices if p.dim() >= 2 and not skip else others).append(p)
        muon = Muon(matrices, lr=lr, weight_decay=weight_decay, momentum=momentum, nesterov=nesterov, ns_steps=ns_steps,
                    adjust_lr_fn=adjust_lr_fn) if matrices else None
        adamw = FusedAdamW([{"params": others, "weight_decay": 0.0}], lr=lr, betas=(0.9, 0.95)) if others else None
        super().__init__(matrices + others, dict(lr=lr, weight_decay=weight_decay), {"muon": muon, "adamw": adamw})
        self.muon, self.adamw = muon, adamw


@OptimizerFactory.register("nora_nadamw")
class NoraNAdamW(CompositeOptimizer):
    optimizer_name = "nora_nadamw"

    def __init__(self, model: nn.Module, lr: float = 3e-4, weight_decay: float = 0.1, nora_lr: float = 5e-3,
                 nora_weight_decay: float = 0.0, nora_beta: float = 0.95, nora_momentum: float = 0.95):
        g = partition_optimizer_parameters(model)
        params = _all_params(g)
        nora = Nora(g.nora, lr=nora_lr, weight_decay=nora_weight_decay, momentum=nora_momentum, beta=nora_beta) if g.nora else None
        rest = _decay_groups(g, weight_decay)
        nadamw = NAdamW(rest, lr=lr) if rest else None
        super().__init__(params, {}, {"nora": nora, "nadamw": nadamw})
        self.nora, self.nadamw = nora, nadamw

    def load_state_dict(self, state_dict):
        if "muon" in state_dict or "adamw" in state_dict:
            raise ValueError("Checkpoint uses muon_adamw state; select optimizer='muon_adamw' to resume it")
        super().load_state_dict(state_dict)


@OptimizerFactory.register("mano_adamw")
class ManoAdamW(CompositeOptimizer):
    optimizer_name = "mano_adamw"

    def __init__(self, model: nn.Module, lr: float = 3e-4, weight_decay: float = 0.1, momentum: float = 0.95, nesterov: bool = True):
        g = partition_optimizer_parameters(model)
        params = _all_params(g)
        mano = Mano(g.nora, lr=lr, weight_decay=weight_decay, momentum=momentum, nesterov=nesterov) if g.nora else None
        rest = _decay_groups(g, weight_decay)
        adamw = FusedAdamW(rest, lr=lr, betas=(0.9, 0.95)) if rest else None
        super().__init__(params, {}, {"mano": mano, "adamw": adamw})
        self.mano, self.adamw = mano, adamw

    def load_state_dict(self, state_dict):
        if "muon" in state_dict or "nora" in state_dict:
            raise ValueError("Checkpoint uses a different optimizer; select the matching --optimizer to resume it")
        super().load_state_dict(state_dict)
