"""FP8 training policy and ops on the tcgen05 ``kind::f8f6f4`` GEMM.

Public surface of the reference's fp8 extension (``astrai/extension/fp8.py:42-406``, ``astrai/extension/ops/fp8.py:55-184``):
``FP8Format`` (E4M3 / E5M2 / HYBRID), the ``DelayedScaling`` / ``DynamicScaling`` recipes
(``scale = amax / FP8_MAX / 2**margin``), per-tensor amax history (:class:`FP8TensorMeta`), ``fp8_autocast(...)``,
``quantize_bf16``, ``mm_fp8``, ``linear_forward_fp8`` / ``linear_backward_fp8``.

Differences in design: the scaling state hangs on the weight tensor itself (``weight._fp8_meta``) instead of a global
table keyed by ``data_ptr``; nothing is patched into ``aten::linear`` - :func:`astrai_b200.ops.linear` asks
:func:`autocast_state` and calls :func:`fp8_linear` when the context is active; the quantise kernel emits the
transposed fp8 copy in the same pass, so the backward GEMMs get K-major operands without ``transpose().contiguous()``
followed by a second quantisation.  On CPU (and for shapes the kernel does not take) the same math runs through
explicit quantise -> fp32 matmul, which is also the oracle of the tests.
"""

from __future__ import annotations

import contextlib
import contextvars
from dataclasses import dataclass
from enum import Enum
from typing import Optional, Tuple

import torch
from torch import Tensor
from torch.autograd import Function

FP8_MAX = {"e4m3": 448.0, "e5m2": 57344.0}
_DTYPES = {"e4m3": torch.float8_e4m3fn, "e5m2": torch.float8_e5m2}


class FP8Format(str, Enum):
    E4M3 = "e4m3"
    E5M2 = "e5m2"
    HYBRID = "hybrid"  # E4M3 for activations / weights, E5M2 for gradients

    def fwd(self) -> str:
        return "e4m3" if self is FP8Format.HYBRID else self.value

    def bwd(self) -> str:
        return "e5m2" if self is FP8Format.HYBRID else self.value


@dataclass
class FP8Recipe:
    history_len: int = 16
    margin: int = 0

    def scale_from_history(self, amax: Tensor, fmt: str) -> Tensor:
        return ((amax.max() / FP8_MAX[fmt]) / (2 ** self.margin)).clamp_min(1e-12)


@dataclass
class DelayedScaling(FP8Recipe):
    """The scale used at step N comes from the largest amax seen in the previous ``history_len`` steps."""

    history_len: int = 16
    margin: int = 0
    measure_first = False


@dataclass
class DynamicScaling(FP8Recipe):
    """The scale comes from the amax of the very tensor being quantised (one extra reduction pass)."""

    history_len: int = 1
    margin: int = 0
    measure_first = True


@dataclass
class BlockScaling(FP8Recipe):
    """One scale per 1 x 128 block of the activations / gradients and per 128 x 128 block of the weights, measured on the
    tensor itself (E4M3 everywhere): no history, no per-layer state.  Served by :mod:`astrai_b200.ops.fp8_block`;
    ``backward`` chooses quantised (``"fp8"``) or bf16 gradient products."""

    history_len: int = 1
    margin: int = 0
    measure_first = True
    backward: str = "fp8"


class FP8TensorMeta:
    """amax rings and current scales of the three operands of one linear layer (weight, input, output gradient)."""

    def __init__(self, device, recipe: FP8Recipe):
        self.recipe = recipe
        n = max(int(recipe.history_len), 1)
        self.hist = {k: torch.ones(n, dtype=torch.float32, device=device) for k in ("w", "x", "g")}
        self.scale = {k: torch.ones(1, dtype=torch.float32, device=device) for k in ("w", "x", "g")}
        self.idx = {"w": 0, "x": 0, "g": 0}
        self.seeded = {"w": False, "x": False, "g": False}

    def seed(self, kind: str, t: Tensor, fmt: str):
        amax = t.detach().abs().amax().float().clamp_min(1e-12)
        self.hist[kind].fill_(amax)
        self.scale[kind].copy_(self.recipe.scale_from_history(self.hist[kind], fmt))
        self.seeded[kind] = True

    def update(self, kind: str, amax: Tensor, fmt: str):
        self.hist[kind][self.idx[kind]] = amax.reshape(())
        self.idx[kind] = (self.idx[kind] + 1) % self.hist[kind].numel()
        self.scale[kind].copy_(self.recipe.scale_from_history(self.hist[kind], fmt))

    # the per-operand spellings of the reference (``astrai/extension/fp8.py:163-187``)
    def update_w(self, amax: Tensor, fmt: str):
        self.update("w", amax, fmt)

    def update_x(self, amax: Tensor, fmt: str):
        self.update("x", amax, fmt)

    def update_g(self, amax: Tensor, fmt: str):
        self.update("g", amax, fmt)

    def init_w(self, t: Tensor, fmt: str):
        self.seed("w", t, fmt)

    def init_x(self, t: Tensor, fmt: str):
        self.seed("x", t, fmt)

    def init_g(self, t: Tensor, fmt: str):
        self.seed("g", t, fmt)

    w_scale = property(lambda self: self.scale["w"])
    x_scale = property(lambda self: self.scale["x"])
    g_scale = property(lambda self: self.scale["g"])


@dataclass
class _AutocastState:
    enabled: bool = False
    recipe: FP8Recipe = None
    fp8_format: FP8Format = FP8Format.HYBRID
    update_interval: int = 1


_PROCESS_WIDE = _AutocastState()  # what holds outside every fp8_autocast block, in every thread (fp8_linear_enable)
_STATE: contextvars.ContextVar[_AutocastState] = contextvars.ContextVar("astrai_b200_fp8", default=_PROCESS_WIDE)


def autocast_state() -> _AutocastState:
    return _STATE.get()


@contextlib.contextmanager
def fp8_autocast(enabled: bool = True, update_interval: int = 1, recipe: Optional[FP8Recipe] = None,
                 fp8_format: FP8Format = FP8Format.HYBRID, margin: int = 0):
    """Run the linear layers inside on fp8 tensor cores (weights and activations quantised per tensor)."""
    recipe = recipe or DelayedScaling(margin=margin)
    token = _STATE.set(_AutocastState(bool(enabled), recipe, FP8Format(fp8_format), int(update_interval)))
    try:
        yield
    finally:
        _STATE.reset(token)


class FP8State:
    """What is in force for fp8 right now, in the shape of the reference's global state object
    (``astrai/extension/fp8.py:190-223``): ``enabled``, ``recipe``, ``fp8_format`` read the innermost
    :func:`fp8_autocast`; scaling state lives on the weights themselves (``get_weight_meta``)."""

    enabled = property(lambda self: autocast_state().enabled)
    recipe = property(lambda self: autocast_state().recipe or DelayedScaling())
    fp8_format = property(lambda self: autocast_state().fp8_format)

    def get_weight_meta(self, w: Tensor) -> FP8TensorMeta:
        return meta_for(w, self.recipe)

    def reset(self, *weights: Tensor) -> None:
        """Forget the scaling history of ``weights`` (their next use seeds it again)."""
        for w in weights:
            if hasattr(w, "_fp8_meta"):
                del w._fp8_meta


def fp8_state() -> FP8State:
    return FP8State()


def fp8_linear_enable(enabled: bool = True, recipe: Optional[FP8Recipe] = None) -> None:
    """Process-wide switch (the reference's ``fp8_linear_enable``, ``astrai/extension/fp8.py:338-345``): linear layers run
    on fp8 wherever no :func:`fp8_autocast` block says otherwise, in every thread."""
    _PROCESS_WIDE.enabled = bool(enabled)
    if recipe is not None or _PROCESS_WIDE.recipe is None:
        _PROCESS_WIDE.recipe = recipe or DelayedScaling()


def fp8_linear_enabled() -> bool:
    return autocast_state().enabled


def meta_for(weight: Tensor, recipe: FP8Recipe) -> FP8TensorMeta:
    meta = getattr(weight, "_fp8_meta", None)
    if meta is None or type(meta.recipe) is not type(recipe) or meta.hist["w"].device != weight.device:
        meta = FP8TensorMeta(weight.device, recipe)
        weight._fp8_meta = meta
    return meta


# --------------------------------------------------------------------------- ops
def _native(x: Tensor) -> bool:
    return x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 2 and x.stride(1) == 1


def quantize_bf16(x: Tensor, scale: Tensor, fmt: str = "e4m3", with_transpose: bool = False):
    """``(q, q_transposed or None, amax)`` with ``q = saturate(x / scale)`` in the given fp8 format."""
    if _native(x):
        from astrai_b200.ops import native

        native.require()
        q, qt, amax = torch.ops.astrai_b200.fp8_quantize(x, scale.reshape(1).float(), fmt == "e5m2", with_transpose)
        return q, (qt if with_transpose else None), amax
    xf = x.float()
    q = (xf / scale.float().clamp_min(1e-30)).clamp(-FP8_MAX[fmt], FP8_MAX[fmt]).to(_DTYPES[fmt])
    return q, (q.t().contiguous() if with_transpose else None), xf.abs().amax().reshape(1)


def mm_fp8(a: Tensor, b: Tensor, scale_a: Tensor, scale_b: Tensor, bias: Optional[Tensor] = None,
           out_dtype=torch.bfloat16) -> Tensor:
    """``(a @ b.T) * scale_a * scale_b (+ bias)`` for fp8 ``a [M,K]``, ``b [N,K]``."""
    if a.is_cuda and a.is_contiguous() and b.is_contiguous() and a.shape[1] % 16 == 0 and out_dtype == torch.bfloat16:
        from astrai_b200.ops import native

        native.require()
        return torch.ops.astrai_b200.fp8_gemm(a, b, scale_a.reshape(1).float(), scale_b.reshape(1).float(),
                                              None if bias is None else bias.to(torch.bfloat16).contiguous())
    out = (a.float() @ b.float().t()) * (scale_a.float() * scale_b.float())
    if bias is not None:
        out = out + bias.float()
    return out.to(out_dtype)


def _scale_for(meta: FP8TensorMeta, kind: str, t: Tensor, fmt: str) -> Tensor:
    if meta.recipe.measure_first or not meta.seeded[kind]:
        meta.seed(kind, t, fmt)
    return meta.scale[kind]


def linear_forward_fp8(x2: Tensor, w: Tensor, bias: Optional[Tensor], meta: FP8TensorMeta, fmt: FP8Format):
    """Returns ``(y, saved)``; ``saved`` carries the transposed fp8 operands the backward pass needs."""
    f = fmt.fwd()
    sx, sw = _scale_for(meta, "x", x2, f), _scale_for(meta, "w", w, f)
    xq, xq_t, ax = quantize_bf16(x2, sx, f, with_transpose=True)
    wq, wq_t, aw = quantize_bf16(w, sw, f, with_transpose=True)
    y = mm_fp8(xq, wq, sx, sw, bias)
    saved = (xq_t, wq_t, sx.clone(), sw.clone())
    if not meta.recipe.measure_first:  # delayed: this step's amax shapes the next step's scale
        meta.update("x", ax, f)
        meta.update("w", aw, f)
    return y, saved


def linear_backward_fp8(gy2: Tensor, saved, meta: FP8TensorMeta, fmt: FP8Format, need_dx: bool = True,
                        need_dw: bool = True) -> Tuple[Optional[Tensor], Optional[Tensor]]:
    xq_t, wq_t, sx, sw = saved
    f = fmt.bwd()
    sg = _scale_for(meta, "g", gy2, f)
    gq, gq_t, ag = quantize_bf16(gy2, sg, f, with_transpose=True)
    dx = mm_fp8(gq, wq_t, sg, sw) if need_dx else None        # [M,N] . [K,N]^T
    dw = mm_fp8(gq_t, xq_t, sg, sx) if need_dw else None      # [N,M] . [K,M]^T
    if not meta.recipe.measure_first:
        meta.update("g", ag, f)
    return dx, dw


class _FP8LinearFn(Function):
    @staticmethod
    def forward(ctx, x: Tensor, w: Tensor, bias: Optional[Tensor], meta: FP8TensorMeta, fmt: FP8Format):
        x2 = x.reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        y, saved = linear_forward_fp8(x2, w, bias, meta, fmt)
        ctx.save_for_backward(*saved)
        ctx.meta, ctx.fmt, ctx.x_shape, ctx.has_bias, ctx.w_ref = meta, fmt, x.shape, bias is not None, w
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, gy: Tensor):
        g2 = gy.reshape(-1, gy.shape[-1]).contiguous()
        dx, dw = linear_backward_fp8(g2, ctx.saved_tensors, ctx.meta, ctx.fmt, ctx.needs_input_grad[0], ctx.needs_input_grad[1])
        db = g2.sum(0) if (ctx.has_bias and ctx.needs_input_grad[2]) else None
        mg = getattr(ctx.w_ref, "main_grad", None)
        if mg is not None and dw is not None:
            mg.add_(dw.float())
            dw = None
        return (dx.view(ctx.x_shape) if dx is not None else None), dw, db, None, None


def fp8_linear(x: Tensor, weight: Tensor, bias: Optional[Tensor] = None) -> Tensor:
    """``x @ weight.T (+ bias)`` on fp8 tensor cores under the active :func:`fp8_autocast` recipe."""
    st = autocast_state()
    recipe = st.recipe or DelayedScaling()
    if isinstance(recipe, BlockScaling):
        from astrai_b200.ops import fp8_block

        if weight.shape[1] % fp8_block.BLOCK == 0:
            return fp8_block.fp8_block_linear(x, weight, bias, backward=recipe.backward)
        recipe = DynamicScaling()  # a width the block kernels do not take: per-tensor scaling measured on the tensor
    return _FP8LinearFn.apply(x, weight, bias, meta_for(weight, recipe), st.fp8_format)


def eligible(x: Tensor, weight: Tensor) -> bool:
    """fp8 takes 2-D-flattenable bf16 CUDA linears whose K and N are multiples of 16."""
    return (x.is_cuda and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and weight.shape[1] % 16 == 0
            and weight.shape[0] % 16 == 0 and (x.numel() // x.shape[-1]) % 16 == 0)


# the reference's names for the same operations (``astrai/extension/fp8.py``, ``astrai/extension/ops/fp8.py``)
fp8_quantize = quantize_bf16
fp8_gemm = mm_fp8
fp8_linear_forward = linear_forward_fp8
fp8_linear_backward = linear_backward_fp8
