"""Differentiable front ends of the sm_100a kernels.

Every function takes the CUDA path when its tensors live on a GPU (the extension must then be loadable: there
is no silent fallback) and the plain-PyTorch statement in :mod:`astrai_b200.ops.reference` on CPU.  The CPU
path is the oracle of the numerics tests.

Gradient of a weight can be returned to autograd (any optimizer works) or, when the parameter carries an fp32
``main_grad`` tensor, accumulated into it by the wgrad kernel itself (``D += dY^T X`` in the GEMM epilogue);
autograd then sees ``None`` for that weight.  The flat-buffer executors install ``main_grad``.
"""

from __future__ import annotations

import contextlib
from typing import Optional, Tuple

import torch
from torch import Tensor
from torch.autograd import Function

from astrai_b200.ops import native, reference

_NATIVE_DTYPES = (torch.bfloat16, torch.float32)


def _use_native(*tensors: Tensor) -> bool:
    t = tensors[0]
    if not t.is_cuda:
        return False
    native.require()
    return all(x.is_cuda and x.dtype in _NATIVE_DTYPES for x in tensors)


def _ops():
    return torch.ops.astrai_b200


def _main_grad(p) -> Optional[Tensor]:
    return getattr(p, "main_grad", None)


# --------------------------------------------------------------------------- GEMM
def _tma_ok(t: Tensor) -> bool:
    return (
        t.dim() == 2 and t.dtype == torch.bfloat16 and t.stride(1) == 1 and t.stride(0) % 8 == 0
        and t.data_ptr() % 16 == 0 and t.stride(0) >= t.size(1)
    )


GEMM_REPACKS = 0  # operands copied into a TMA-addressable layout since import (a non-zero value in a hot loop is a layout bug)


def _tma_repack(t: Tensor) -> Tensor:
    """A copy of 2-D ``t`` that TMA can address: unit inner stride, 16-byte aligned base, row stride a multiple of 8
    elements.  The copy keeps the logical shape (the padding lives in the row stride only)."""
    global GEMM_REPACKS
    GEMM_REPACKS += 1
    rows, cols = t.shape
    buf = torch.zeros((rows, -(-cols // 8) * 8), dtype=torch.bfloat16, device=t.device)
    view = buf[:, :cols]
    view.copy_(t)
    return view


def gemm(a: Tensor, b: Tensor, out: Optional[Tensor] = None, a_kmajor: bool = True, b_kmajor: bool = True,
         out_f32: bool = False, accumulate: bool = False) -> Tensor:
    """``D[M,N] (+)= op(A) @ op(B)`` on tcgen05.

    ``a`` is stored ``[M,K]`` (``a_kmajor``) or ``[K,M]``; ``b`` is stored ``[N,K]`` (``b_kmajor``) or ``[K,N]``.
    On CUDA the product always runs on the tcgen05 kernel: an operand that TMA cannot address (unaligned base, row
    stride not a multiple of 8 elements, strided inner dimension) is first copied into an addressable layout (counted
    in ``GEMM_REPACKS``), and a non-bf16 operand is an error.  The plain-PyTorch statement below is the CPU path.
    """
    if a.is_cuda:
        if a.dtype != torch.bfloat16 or b.dtype != torch.bfloat16 or a.dim() != 2 or b.dim() != 2:
            raise TypeError("ops.gemm on CUDA takes 2-D bf16 operands")
        native.require()
        a = a if _tma_ok(a) else _tma_repack(a)
        b = b if _tma_ok(b) else _tma_repack(b)
        if out is not None and out.stride(-1) != 1:
            tmp = _ops().gemm(a, b, None, a_kmajor, b_kmajor, out_f32, False)
            if accumulate:
                out.add_(tmp)
            else:
                out.copy_(tmp)
            return out
        return _ops().gemm(a, b, out, a_kmajor, b_kmajor, out_f32, accumulate)
    lhs = a if a_kmajor else a.t()
    rhs = b.t() if b_kmajor else b
    res = (lhs.float() @ rhs.float()).to(torch.float32 if out_f32 else a.dtype)
    if out is None:
        return res
    if accumulate:
        out.add_(res)
    else:
        out.copy_(res)
    return out


class _LinearFn(Function):
    @staticmethod
    def forward(ctx, x: Tensor, w: Tensor, bias: Optional[Tensor], w_ref):
        # w_ref: the object that may carry `main_grad` (the Parameter, or a fused view installed by an executor)
        x2 = x.reshape(-1, x.shape[-1])
        y = gemm(x2, w)
        if bias is not None:
            y = y + bias
        ctx.save_for_backward(x2, w)
        ctx.has_bias = bias is not None
        ctx.w_ref = w_ref
        ctx.x_shape = x.shape
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, gy: Tensor):
        x2, w = ctx.saved_tensors
        g2 = gy.reshape(-1, gy.shape[-1])
        if not g2.is_contiguous():
            g2 = g2.contiguous()
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = gemm(g2, w, a_kmajor=True, b_kmajor=False).view(ctx.x_shape)  # dY[M,N] @ W[N,K]
        mg = _main_grad(ctx.w_ref)
        if mg is not None:
            gemm(g2, x2, out=mg, a_kmajor=False, b_kmajor=False, out_f32=True, accumulate=True)  # dY^T @ X
        elif ctx.needs_input_grad[1]:
            dw = gemm(g2, x2, a_kmajor=False, b_kmajor=False)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = g2.sum(0)
        return dx, dw, db, None


def linear(x: Tensor, weight: Tensor, bias: Optional[Tensor] = None, grad_owner=None) -> Tensor:
    """``x @ weight.T (+ bias)``.  ``grad_owner`` overrides where the wgrad kernel looks for ``main_grad``."""
    from astrai_b200.ops import fp8

    if fp8.autocast_state().enabled and (fp8.eligible(x, weight) or not x.is_cuda):
        return fp8.fp8_linear(x, weight, bias)
    if x.is_cuda and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16:
        native.require()
        return _LinearFn.apply(x, weight, bias, grad_owner if grad_owner is not None else weight)
    return reference.linear(x, weight, bias)


# --------------------------------------------------------------------------- RMSNorm
class _RMSNormFn(Function):
    @staticmethod
    def forward(ctx, x: Tensor, w: Tensor, eps: float):
        xc = x.contiguous()
        y, rstd = _ops().rmsnorm_fwd(xc, w.contiguous(), eps)
        ctx.save_for_backward(xc, w, rstd)
        ctx.w_ref = w
        return y

    @staticmethod
    def backward(ctx, gy: Tensor):
        x, w, rstd = ctx.saved_tensors
        dx, dw = _ops().rmsnorm_bwd(gy.contiguous(), x, w.contiguous(), rstd)
        mg = _main_grad(ctx.w_ref)
        if mg is not None:
            mg.add_(dw)
            return dx, None, None
        return dx, dw.to(w.dtype), None


def rms_norm(x: Tensor, weight: Tensor, eps: float) -> Tensor:
    if _use_native(x, weight) and x.dtype == weight.dtype:
        return _RMSNormFn.apply(x, weight, float(eps))
    return reference.rms_norm(x, weight, eps)


class _AddRMSNormFn(Function):
    """``s = x + res; y = rms_norm(s)`` in one pass over the rows; the backward adds the gradient that reaches ``s``
    directly (the residual branch) into the norm's input gradient inside the same kernel."""

    @staticmethod
    def forward(ctx, x: Tensor, res: Tensor, w: Tensor, eps: float):
        s, y, rstd = _ops().add_rmsnorm_fwd(x.contiguous(), res.contiguous(), w.contiguous(), eps)
        ctx.save_for_backward(s, w, rstd)
        ctx.w_ref = w
        return s, y

    @staticmethod
    def backward(ctx, gs: Tensor, gy: Tensor):
        s, w, rstd = ctx.saved_tensors
        if gy is None:
            return gs, gs, None, None
        if gs is None:
            dx, dw = _ops().rmsnorm_bwd(gy.contiguous(), s, w.contiguous(), rstd)
        else:
            dx, dw = _ops().rmsnorm_bwd_add(gy.contiguous(), s, w.contiguous(), rstd, gs.contiguous())
        mg = _main_grad(ctx.w_ref)
        if mg is not None:
            mg.add_(dw)
            return dx, dx, None, None
        return dx, dx, dw.to(w.dtype), None


def add_rms_norm(x: Tensor, res: Tensor, weight: Tensor, eps: float) -> Tuple[Tensor, Tensor]:
    """``(x + res, rms_norm(x + res, weight))``: the residual add of a pre-norm block fused into the norm that follows it
    (reference: ``astrai/model/components/decoder_block.py:67-68`` does the add and the norm as two ops)."""
    cols = x.shape[-1]
    if (_use_native(x, res, weight) and x.dtype == weight.dtype == res.dtype and x.shape == res.shape
            and cols % 8 == 0 and 512 <= cols <= 16384):
        return _AddRMSNormFn.apply(x, res, weight, float(eps))
    s = x + res
    return s, rms_norm(s, weight, eps)


# --------------------------------------------------------------------------- RoPE
def _as_tokens(x: Tensor) -> Tensor:
    """[..., H, D] -> [T, H, D] without a copy when the leading dims collapse."""
    h, d = x.shape[-2:]
    try:
        return x.view(-1, h, d)
    except RuntimeError:
        return x.reshape(-1, h, d)


def _rope_native_ok(x: Tensor, freqs: Tensor) -> bool:
    return (
        _use_native(x) and freqs.is_cuda and x.shape[-1] % 8 == 0 and x.stride(-1) == 1
        and freqs.shape[-1] == 2 and freqs.shape[-2] * 2 == x.shape[-1]
    )


def _rope_kernel(x3: Tensor, out3: Tensor, freqs: Tensor, inverse: bool):
    ok = all(s % 8 == 0 for s in (x3.stride(0), x3.stride(1), out3.stride(0), out3.stride(1)))
    if not ok or x3.data_ptr() % 16 or out3.data_ptr() % 16:
        x3 = x3.contiguous()
    _ops().rope(x3, out3, freqs, inverse)


class _RopeFn(Function):
    @staticmethod
    def forward(ctx, x: Tensor, freqs: Tensor):
        x3 = _as_tokens(x)
        f = freqs.reshape(-1, freqs.shape[-2], 2).float().contiguous()
        out = torch.empty(x3.shape, dtype=x.dtype, device=x.device)
        _rope_kernel(x3, out, f, False)
        ctx.save_for_backward(f)
        ctx.shape = x.shape
        return out.view(x.shape)

    @staticmethod
    def backward(ctx, gy: Tensor):
        (f,) = ctx.saved_tensors
        g3 = _as_tokens(gy.contiguous())
        out = torch.empty_like(g3)
        _rope_kernel(g3, out, f, True)
        return out.view(ctx.shape), None


def rotary(x: Tensor, freqs: Tensor) -> Tensor:
    """Rotate adjacent pairs ``(x[2i], x[2i+1])`` by the (cos, sin) rows of ``freqs``.

    ``x`` is ``[..., H, D]``; ``freqs`` is ``[..., D/2, 2]`` fp32 with the same leading shape.
    Reference semantics: ``astrai/extension/backend/rotary.py:25-33``.
    """
    if _rope_native_ok(x, freqs):
        return _RopeFn.apply(x, freqs)
    return reference.rotary(x, freqs)


class _QKVRopeFn(Function):
    """Split a fused projection ``[T, (Hq+2Hkv)*D]`` into rotated q, rotated k and v (all contiguous)."""

    @staticmethod
    def forward(ctx, qkv: Tensor, freqs: Tensor, hq: int, hkv: int, d: int):
        t = qkv.shape[0]
        qkv3 = qkv.view(t, hq + 2 * hkv, d)
        f = freqs.reshape(-1, d // 2, 2).float().contiguous()
        q = torch.empty((t, hq, d), dtype=qkv.dtype, device=qkv.device)
        k = torch.empty((t, hkv, d), dtype=qkv.dtype, device=qkv.device)
        _ops().rope(qkv3[:, :hq], q, f, False)
        _ops().rope(qkv3[:, hq:hq + hkv], k, f, False)
        v = qkv3[:, hq + hkv:].contiguous()
        ctx.save_for_backward(f)
        ctx.dims = (hq, hkv, d)
        return q, k, v

    @staticmethod
    def backward(ctx, gq: Tensor, gk: Tensor, gv: Tensor):
        (f,) = ctx.saved_tensors
        hq, hkv, d = ctx.dims
        t = gq.shape[0]
        g = torch.empty((t, hq + 2 * hkv, d), dtype=gq.dtype, device=gq.device)
        _ops().rope(gq.contiguous(), g[:, :hq], f, True)
        _ops().rope(gk.contiguous(), g[:, hq:hq + hkv], f, True)
        g[:, hq + hkv:].copy_(gv)
        return g.view(t, -1), None, None, None, None


def qkv_rope(qkv: Tensor, freqs: Tensor, hq: int, hkv: int, d: int) -> Tuple[Tensor, Tensor, Tensor]:
    """``qkv`` is ``[T, (hq+2*hkv)*d]``; returns rotated q ``[T,hq,d]``, rotated k and v ``[T,hkv,d]``."""
    if _use_native(qkv) and freqs.is_cuda and d % 8 == 0 and qkv.is_contiguous():
        return _QKVRopeFn.apply(qkv, freqs, hq, hkv, d)
    t = qkv.shape[0]
    qkv3 = qkv.view(t, hq + 2 * hkv, d)
    f = freqs.reshape(t, d // 2, 2)
    return reference.rotary(qkv3[:, :hq], f), reference.rotary(qkv3[:, hq:hq + hkv], f), qkv3[:, hq + hkv:]


# --------------------------------------------------------------------------- SwiGLU
class _SwiGLUFn(Function):
    @staticmethod
    def forward(ctx, gate: Tensor, up: Tensor):
        ctx.save_for_backward(gate, up)
        return _ops().swiglu_fwd(gate, up)

    @staticmethod
    def backward(ctx, gy: Tensor):
        gate, up = ctx.saved_tensors
        d = _ops().swiglu_bwd(gy.contiguous(), gate, up)
        f = gate.shape[1]
        return d[:, :f], d[:, f:]


class _SwiGLUFusedFn(Function):
    @staticmethod
    def forward(ctx, gu: Tensor):
        f = gu.shape[1] // 2
        ctx.save_for_backward(gu)
        return _ops().swiglu_fwd(gu[:, :f], gu[:, f:])

    @staticmethod
    def backward(ctx, gy: Tensor):
        (gu,) = ctx.saved_tensors
        f = gu.shape[1] // 2
        return _ops().swiglu_bwd(gy.contiguous(), gu[:, :f], gu[:, f:])


def swiglu(gate: Tensor, up: Tensor) -> Tensor:
    """``up * silu(gate)`` (reference: ``astrai/model/components/mlp.py:41``)."""
    if _use_native(gate, up) and gate.shape[-1] % 8 == 0 and gate.dtype == up.dtype:
        shape = gate.shape
        g2, u2 = gate.reshape(-1, shape[-1]), up.reshape(-1, shape[-1])
        if g2.stride() != u2.stride() or g2.stride(1) != 1 or g2.stride(0) % 8:
            g2, u2 = g2.contiguous(), u2.contiguous()
        return _SwiGLUFn.apply(g2, u2).view(shape)
    return reference.swiglu(gate, up)


def swiglu_fused(gate_up: Tensor) -> Tensor:
    """Input ``[..., 2F]`` with the gate in columns ``[0,F)`` and the up projection in ``[F,2F)``."""
    f = gate_up.shape[-1] // 2
    if _use_native(gate_up) and f % 8 == 0 and gate_up.is_contiguous():
        shape = gate_up.shape
        return _SwiGLUFusedFn.apply(gate_up.view(-1, 2 * f)).view(*shape[:-1], f)
    return reference.swiglu(gate_up[..., :f], gate_up[..., f:])


# --------------------------------------------------------------------------- Embedding
class _EmbeddingFn(Function):
    @staticmethod
    def forward(ctx, ids: Tensor, table: Tensor):
        ctx.save_for_backward(ids)
        ctx.table = table
        return _ops().embedding_fwd(ids.contiguous(), table)

    @staticmethod
    def backward(ctx, gy: Tensor):
        (ids,) = ctx.saved_tensors
        table = ctx.table
        # Sorted segmented reduce: rows of equal ids are summed in a fixed order by one CTA each, so the gradient of a
        # tied embedding / lm_head weight is the same bits on every run (an atomic scatter-add is not).
        sorted_ids, perm = torch.sort(ids.reshape(-1), stable=True)
        g2 = gy.reshape(-1, gy.shape[-1]).contiguous()
        mg = _main_grad(table)
        if mg is not None:
            _ops().embedding_bwd_sorted_(sorted_ids, perm, g2, mg)
            return None, None
        acc = torch.zeros(table.shape, dtype=torch.float32, device=table.device)
        _ops().embedding_bwd_sorted_(sorted_ids, perm, g2, acc)
        return None, acc.to(table.dtype)


def embedding(ids: Tensor, table: Tensor) -> Tensor:
    if _use_native(table) and ids.is_cuda and ids.dtype == torch.long and table.shape[1] % 8 == 0 and table.is_contiguous():
        return _EmbeddingFn.apply(ids, table)
    return torch.nn.functional.embedding(ids, table)


# --------------------------------------------------------------------------- losses
_LOSS_GRAD = {"scale": None, "denominator": None}


@contextlib.contextmanager
def assume_loss_grad(scale: Optional[float]):
    """Promise that the loss computed inside will be back-propagated with exactly ``d loss = scale``.

    The fused linear + cross-entropy then folds the scale into the gradients it produces during the forward
    pass and accumulates the weight gradient straight into ``main_grad``; its backward ignores the incoming
    gradient value.  Without the promise it keeps an fp32 temporary and scales it in backward.
    """
    prev = _LOSS_GRAD["scale"]
    _LOSS_GRAD["scale"] = scale
    try:
        yield
    finally:
        _LOSS_GRAD["scale"] = prev


@contextlib.contextmanager
def loss_denominator(count: Optional[Tensor]):
    """Inside, a mean cross-entropy divides its sum by ``count`` (a scalar tensor) instead of by the number of targets it
    is given.  For a rank that holds a slice of a batch's tokens and whose gradients are then averaged over the ranks of
    the slice group: with ``count`` = trained tokens of the whole batch / ranks, the average of the ranks' losses (and
    gradients) is the mean over all trained tokens, however unevenly they fall on the slices.  ``None`` changes nothing."""
    prev = _LOSS_GRAD["denominator"]
    _LOSS_GRAD["denominator"] = count
    try:
        yield
    finally:
        _LOSS_GRAD["denominator"] = prev


def _mean_denominator(targets: Tensor, ignore_index: int) -> Tensor:
    count = _LOSS_GRAD["denominator"]
    if count is not None:
        return count.to(device=targets.device, dtype=torch.float32).reshape(()).clamp(min=1e-6)
    return (targets != ignore_index).sum().clamp(min=1).float()


def cross_entropy(logits: Tensor, targets: Tensor, label_smoothing: float = 0.0, ignore_index: int = -100,
                  reduction: str = "mean") -> Tensor:
    """Cross-entropy over the last dim of ``logits`` (any leading shape), fp32 math.

    Matches ``F.cross_entropy(logits.float(), ...)`` as the reference strategies call it
    (``astrai/trainer/strategy.py:336-340``, ``:385-390``).  Not fused with the projection; see
    :func:`linear_cross_entropy` for the path that never stores fp32 logits.
    """
    v = logits.shape[-1]
    rows = reference.cross_entropy_rows(logits.reshape(-1, v), targets.reshape(-1), label_smoothing, ignore_index)
    if reduction == "none":
        return rows.view(targets.shape)
    if reduction == "sum":
        return rows.sum()
    return rows.sum() / _mean_denominator(targets.reshape(-1), ignore_index)


class _LinearCEFn(Function):
    @staticmethod
    def forward(ctx, h: Tensor, w: Tensor, targets: Tensor, smoothing: float, ignore_index: int, chunk: int, w_ref):
        t, d = h.shape
        n_valid = _mean_denominator(targets, ignore_index)
        baked = _LOSS_GRAD["scale"]
        need_grad = ctx.needs_input_grad[0] or ctx.needs_input_grad[1]
        gscale = ((baked if baked is not None else 1.0) / n_valid).reshape(1).contiguous()
        mg = _main_grad(w_ref)
        direct = need_grad and baked is not None and mg is not None
        dh = torch.empty_like(h) if need_grad else None
        dw_tmp = None
        if need_grad and not direct:
            dw_tmp = torch.zeros(w.shape, dtype=torch.float32, device=w.device)
        loss_sum = torch.zeros((), dtype=torch.float32, device=h.device)
        for s in range(0, t, chunk):
            hc = h[s:s + chunk]
            logits = gemm(hc, w)  # [c, V] bf16, consumed and overwritten below
            rows, _ = _ops().ce_rows(logits, targets[s:s + chunk].contiguous(), smoothing, ignore_index, gscale, need_grad)
            loss_sum += rows.sum()
            if need_grad:
                gemm(logits, w, out=dh[s:s + chunk], a_kmajor=True, b_kmajor=False)
                gemm(logits, hc, out=mg if direct else dw_tmp, a_kmajor=False, b_kmajor=False, out_f32=True, accumulate=True)
        ctx.baked = baked is not None
        ctx.direct = direct
        ctx.w_ref = w_ref
        ctx.w_dtype = w.dtype
        if need_grad:
            ctx.save_for_backward(dh, dw_tmp) if dw_tmp is not None else ctx.save_for_backward(dh)
        return loss_sum / n_valid

    @staticmethod
    def backward(ctx, g: Tensor):
        saved = ctx.saved_tensors
        dh = saved[0]
        dw_tmp = saved[1] if len(saved) > 1 else None
        if not ctx.baked:
            dh = dh * g.to(dh.dtype)
        dw = None
        if dw_tmp is not None:
            mg = _main_grad(ctx.w_ref)
            if mg is not None:
                if ctx.baked:
                    mg.add_(dw_tmp)
                else:
                    mg.addcmul_(dw_tmp, g.float())
            else:
                dw = (dw_tmp if ctx.baked else dw_tmp * g.float()).to(ctx.w_dtype)
        return dh, dw, None, None, None, None, None


def linear_cross_entropy(h: Tensor, weight: Tensor, targets: Tensor, label_smoothing: float = 0.0,
                         ignore_index: int = -100, chunk_tokens: int = 8192, grad_owner=None) -> Tensor:
    """Mean cross-entropy of ``h @ weight.T`` against ``targets`` without keeping ``[T, V]`` logits.

    Works chunk by chunk over tokens: project (tcgen05 GEMM, bf16 logits), reduce each row to its loss and
    overwrite the chunk with its gradient, then immediately run dgrad and wgrad for the chunk.  Replaces
    ``lm_head`` + ``F.cross_entropy`` of the reference (``astrai/trainer/strategy.py:330-347``).
    """
    h2 = h.reshape(-1, h.shape[-1])
    t2 = targets.reshape(-1)
    if h2.is_cuda and h2.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16:
        native.require()
        return _LinearCEFn.apply(h2.contiguous(), weight, t2, float(label_smoothing), int(ignore_index),
                                 int(chunk_tokens), grad_owner if grad_owner is not None else weight)
    logits = reference.linear(h2, weight)
    return cross_entropy(logits, t2, label_smoothing, ignore_index)


class _LinearLogprobFn(Function):
    @staticmethod
    def forward(ctx, h: Tensor, w: Tensor, ids: Tensor, chunk: int, w_ref):
        t = h.shape[0]
        out = torch.empty(t, dtype=torch.float32, device=h.device)
        for s in range(0, t, chunk):
            logits = gemm(h[s:s + chunk], w)
            _, lp = _ops().ce_rows(logits, ids[s:s + chunk].contiguous(), 0.0, -100, None, False)
            out[s:s + chunk] = lp
        ctx.save_for_backward(h, w, ids, out)
        ctx.chunk = chunk
        ctx.w_ref = w_ref
        return out

    @staticmethod
    def backward(ctx, g: Tensor):
        h, w, ids, lp = ctx.saved_tensors
        t = h.shape[0]
        g = g.float().contiguous()
        dh = torch.empty_like(h)
        mg = _main_grad(ctx.w_ref)
        dw_acc = mg if mg is not None else torch.zeros(w.shape, dtype=torch.float32, device=w.device)
        for s in range(0, t, ctx.chunk):
            hc = h[s:s + ctx.chunk]
            logits = gemm(hc, w)  # recomputed: the forward kept no logits
            _ops().logprob_bwd_(logits, ids[s:s + ctx.chunk].contiguous(), lp[s:s + ctx.chunk].contiguous(), g[s:s + ctx.chunk].contiguous())
            gemm(logits, w, out=dh[s:s + ctx.chunk], a_kmajor=True, b_kmajor=False)
            gemm(logits, hc, out=dw_acc, a_kmajor=False, b_kmajor=False, out_f32=True, accumulate=True)
        return dh, (None if mg is not None else dw_acc.to(w.dtype)), None, None, None


def linear_token_logprobs(h: Tensor, weight: Tensor, ids: Tensor, chunk_tokens: int = 8192, grad_owner=None) -> Tensor:
    """``log_softmax(h @ weight.T)[ids]`` per token in fp32, logits never kept (DPO / GRPO; reference
    ``astrai/trainer/strategy.py:66-70``)."""
    shape = ids.shape
    h2 = h.reshape(-1, h.shape[-1])
    i2 = ids.reshape(-1)
    if h2.is_cuda and h2.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16:
        native.require()
        return _LinearLogprobFn.apply(h2.contiguous(), weight, i2, int(chunk_tokens),
                                      grad_owner if grad_owner is not None else weight).view(shape)
    return reference.token_logprobs(reference.linear(h2, weight), i2).view(shape)


# --------------------------------------------------------------------------- optimizer helpers
def sumsq(x: Tensor, out: Optional[Tensor] = None) -> Tensor:
    """``out[0] += sum(x**2)`` in fp32 (``out`` created as zero when omitted)."""
    if out is None:
        out = torch.zeros(1, dtype=torch.float32, device=x.device)
    if _use_native(x):
        _ops().sumsq_(x.contiguous().view(-1), out)
    else:
        out += x.float().pow(2).sum()
    return out


def clip_coef(sumsq_t: Tensor, max_norm: Optional[float], pre_scale: float = 1.0) -> Tuple[Tensor, Tensor]:
    """(coef, norm): ``norm = sqrt(sumsq) * pre_scale`` and ``coef = min(1, max_norm/(norm+1e-6)) * pre_scale``."""
    mx = float(max_norm) if max_norm is not None else -1.0
    if sumsq_t.is_cuda:
        native.require()
        coef = torch.empty(1, dtype=torch.float32, device=sumsq_t.device)
        norm = torch.empty(1, dtype=torch.float32, device=sumsq_t.device)
        _ops().clip_coef_(sumsq_t, mx, float(pre_scale), coef, norm)
        return coef, norm
    norm = sumsq_t.sqrt() * pre_scale
    coef = torch.ones_like(norm) if mx <= 0 else (mx / (norm + 1e-6)).clamp(max=1.0)
    return coef * pre_scale, norm


def adamw_(p: Tensor, grad: Tensor, exp_avg: Tensor, exp_avg_sq: Tensor, *, lr: float, betas=(0.9, 0.999),
           eps: float = 1e-8, weight_decay: float = 0.01, step: int, master: Optional[Tensor] = None,
           grad_scale: Optional[Tensor] = None, zero_grad: bool = False):
    """One decoupled-weight-decay Adam step on flat buffers (fp32 gradient and moments)."""
    b1, b2 = betas
    if p.is_cuda:
        native.require()
        _ops().adamw_(p, master, grad, exp_avg, exp_avg_sq, lr, b1, b2, eps, weight_decay, step, grad_scale, zero_grad)
        return
    g = grad if grad_scale is None else grad * grad_scale
    w = master if master is not None else p.float()
    exp_avg.mul_(b1).add_(g, alpha=1 - b1)
    exp_avg_sq.mul_(b2).addcmul_(g, g, value=1 - b2)
    bc1 = 1 - b1 ** step
    bc2 = 1 - b2 ** step
    w = w * (1 - lr * weight_decay) - (lr / bc1) * exp_avg / (exp_avg_sq.sqrt() / bc2 ** 0.5 + eps)
    if master is not None:
        master.copy_(w)
    p.copy_(w.to(p.dtype))
    if zero_grad:
        grad.zero_()
