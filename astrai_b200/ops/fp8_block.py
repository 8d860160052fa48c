"""Block-scaled fp8 (E4M3): one fp32 scale per 1 x 128 block of the activations and per 128 x 128 block of the weights.

Finer scales than the per-tensor recipe of ``ops/fp8.py`` keep outlier channels from flattening everything else; the
GEMM (``ops/csrc/gemm_fp8_block.cu``) runs each 128-wide K block into a fresh tensor-memory accumulator and promotes the
partial sums with ``sa[m, kb] * sb[n / 128, kb]`` in registers.  :func:`fp8_block_linear` quantises the forward product
and, where the shapes allow (the contraction sizes of the two gradient products - the layer's output width and the token
count - are multiples of 128), both gradient products as well: the operand that is contracted over its rows is
transposed first and quantised along its new rows, so all three products run on the one block GEMM.  Other shapes, and
``backward="bf16"``, take bf16 gradients from the saved high-precision operands.  ``fp8_autocast(recipe=BlockScaling())``
routes every eligible linear layer here.  The reference's fp8 path is per-tensor only
(``astrai/extension/fp8.py:61-105``; ``csrc/kernels/fp8/mm.cu:49-54``).
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch
from torch import Tensor, nn

from astrai_b200.ops import native

BLOCK = 128
E4M3_MAX = 448.0


def eligible(x: Tensor, in_features: int) -> bool:
    return x.is_cuda and x.dtype == torch.bfloat16 and in_features % BLOCK == 0 and native.is_available()


def quantize_act_block_reference(x: Tensor) -> Tuple[Tensor, Tensor]:
    """``(q [R, C] float8_e4m3fn, sa_t [C / 128, R] fp32)``: PyTorch statement of the kernel (CPU path, tests)."""
    r, c = x.shape
    blocks = x.float().view(r, c // BLOCK, BLOCK)
    amax = blocks.abs().amax(dim=-1)
    scale = torch.where(amax > 0, amax / E4M3_MAX, torch.ones_like(amax))
    q = (blocks / scale[..., None]).clamp(-E4M3_MAX, E4M3_MAX).view(r, c).to(torch.float8_e4m3fn)
    return q, scale.t().contiguous()


def quantize_weight_block_reference(w: Tensor) -> Tuple[Tensor, Tensor]:
    """``(q [N, K] float8_e4m3fn, sb [ceil(N / 128), K / 128] fp32)``."""
    n, k = w.shape
    nb = -(-n // BLOCK)
    padded = torch.zeros(nb * BLOCK, k, dtype=torch.float32, device=w.device)
    padded[:n] = w.float()
    blocks = padded.view(nb, BLOCK, k // BLOCK, BLOCK)
    amax = blocks.abs().amax(dim=(1, 3))
    scale = torch.where(amax > 0, amax / E4M3_MAX, torch.ones_like(amax))
    q = (blocks / scale[:, None, :, None]).clamp(-E4M3_MAX, E4M3_MAX).view(nb * BLOCK, k)[:n].to(torch.float8_e4m3fn)
    return q, scale


def quantize_act_block(x: Tensor) -> Tuple[Tensor, Tensor]:
    if x.is_cuda:
        native.require()
        return torch.ops.astrai_b200.fp8_quantize_block(x.contiguous(), False)
    return quantize_act_block_reference(x)


def quantize_weight_block(w: Tensor) -> Tuple[Tensor, Tensor]:
    if w.is_cuda:
        native.require()
        return torch.ops.astrai_b200.fp8_quantize_block(w.contiguous(), True)
    return quantize_weight_block_reference(w)


def dequantize_act(q: Tensor, sa_t: Tensor) -> Tensor:
    r, c = q.shape
    return (q.float().view(r, c // BLOCK, BLOCK) * sa_t.t()[..., None]).view(r, c)


def dequantize_weight(q: Tensor, sb: Tensor) -> Tensor:
    n, k = q.shape
    rows = torch.arange(n, device=q.device) // BLOCK
    return (q.float().view(n, k // BLOCK, BLOCK) * sb[rows][..., None]).view(n, k)


def mm_fp8_block(a_q: Tensor, sa_t: Tensor, b_q: Tensor, sb: Tensor, bias: Optional[Tensor] = None) -> Tensor:
    """``sum_kb sa * sb * (A_kb @ B_kb.T)`` as bf16; ``a_q [M, K]``, ``b_q [N, K]``."""
    if a_q.is_cuda:
        native.require()
        return torch.ops.astrai_b200.fp8_gemm_block(a_q.contiguous(), sa_t.contiguous(), b_q.contiguous(), sb.contiguous(),
                                                    None if bias is None else bias.to(torch.bfloat16).contiguous())
    out = dequantize_act(a_q, sa_t) @ dequantize_weight(b_q, sb).t()
    if bias is not None:
        out = out + bias.float()
    return out.to(torch.bfloat16)


def _block_product(a: Tensor, b: Tensor) -> Tensor:
    """``a [M, K] @ b [N, K].T`` with ``a`` quantised per 1 x 128 block and ``b`` per 128 x 128 block (bf16 result)."""
    a_q, sa_t = quantize_act_block(a)
    b_q, sb = quantize_weight_block(b)
    return mm_fp8_block(a_q, sa_t, b_q, sb)


class _Fp8BlockLinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: Tensor, w: Tensor, bias: Optional[Tensor], backward: str):
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        a_q, sa_t = quantize_act_block(x2)
        b_q, sb = quantize_weight_block(w)
        ctx.save_for_backward(x2, w)
        ctx.has_bias, ctx.shape, ctx.mode, ctx.w_ref = bias is not None, shape, backward, w
        return mm_fp8_block(a_q, sa_t, b_q, sb, bias).view(*shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, gy: Tensor):
        x2, w = ctx.saved_tensors
        g2 = gy.reshape(-1, gy.shape[-1])
        m, n = g2.shape
        quantised = ctx.mode == "fp8" and n % BLOCK == 0 and m % BLOCK == 0
        gx = gw = None
        if ctx.needs_input_grad[0]:
            if quantised:  # dX [M, K] = dY [M, N] @ W [N, K]: contraction over N, the second operand is W^T [K, N]
                gx = _block_product(g2.to(torch.bfloat16).contiguous(), w.to(torch.bfloat16).t().contiguous()).to(g2.dtype)
            else:
                gx = g2 @ w.to(g2.dtype)
            gx = gx.view(ctx.shape)
        if ctx.needs_input_grad[1]:
            if quantised:  # dW [N, K] = dY^T [N, M] @ X [M, K]: contraction over M, operands dY^T and X^T [K, M]
                gw = _block_product(g2.to(torch.bfloat16).t().contiguous(), x2.to(torch.bfloat16).t().contiguous())
            else:
                gw = g2.t() @ x2.to(g2.dtype)
            mg = getattr(ctx.w_ref, "main_grad", None)
            if mg is not None:  # the flat runtime's fp32 gradient buffer
                mg.add_(gw.float())
                gw = None
            else:
                gw = gw.to(w.dtype)
        gb = g2.sum(0) if ctx.has_bias and ctx.needs_input_grad[2] else None
        return gx, gw, gb, None


def fp8_block_linear(x: Tensor, weight: Tensor, bias: Optional[Tensor] = None, backward: str = "fp8") -> Tensor:
    """``x @ weight.T`` with both operands quantised block-wise on the fly.  ``backward="fp8"`` (default) quantises the two
    gradient products the same way when their contraction sizes are multiples of 128; ``"bf16"`` keeps them in bf16."""
    if backward not in ("fp8", "bf16"):
        raise ValueError("backward must be 'fp8' or 'bf16'")
    return _Fp8BlockLinearFn.apply(x, weight, bias, backward)


class Fp8BlockLinear(nn.Module):
    """Inference layer with the weight quantised once (128 x 128 blocks) and the activations per call (1 x 128)."""

    def __init__(self, in_features: int, out_features: int, bias: bool = False, device=None):
        super().__init__()
        if in_features % BLOCK:
            raise ValueError("in_features must be a multiple of 128")
        self.in_features, self.out_features = in_features, out_features
        self.register_buffer("weight_q", torch.zeros(out_features, in_features, dtype=torch.float8_e4m3fn, device=device))
        self.register_buffer("weight_scale", torch.ones(-(-out_features // BLOCK), in_features // BLOCK, dtype=torch.float32, device=device))
        self.register_buffer("bias", torch.zeros(out_features, dtype=torch.bfloat16, device=device) if bias else None)

    @classmethod
    def from_linear(cls, linear: nn.Module) -> "Fp8BlockLinear":
        w = linear.weight.detach()
        b = getattr(linear, "bias", None)
        out = cls(w.shape[1], w.shape[0], bias=b is not None, device=w.device)
        q, s = quantize_weight_block(w.to(torch.bfloat16))
        out.weight_q.copy_(q)
        out.weight_scale.copy_(s)
        if b is not None:
            out.bias.copy_(b.detach().to(torch.bfloat16))
        return out

    def forward(self, x: Tensor) -> Tensor:
        shape = x.shape
        a_q, sa_t = quantize_act_block(x.to(torch.bfloat16).reshape(-1, shape[-1]))
        return mm_fp8_block(a_q, sa_t, self.weight_q, self.weight_scale, self.bias).view(*shape[:-1], self.out_features)
