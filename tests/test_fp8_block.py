"""Block-scaled fp8: the quantisers and the GEMM against explicit dequantise -> fp32 matmul."""

import pytest
import torch

from astrai_b200.ops import fp8_block as fb


def test_reference_quantisers_roundtrip_cpu():
    torch.manual_seed(0)
    x = torch.randn(5, 256) * torch.tensor([1.0, 50.0]).repeat_interleave(128)  # one loud block per row
    q, sa_t = fb.quantize_act_block(x.bfloat16())
    assert q.shape == (5, 256) and sa_t.shape == (2, 5)
    back = fb.dequantize_act(q, sa_t)
    assert ((back - x.bfloat16().float()).abs() <= 0.07 * x.abs().view(5, 2, 128).amax(-1).repeat_interleave(128, 1)).all()
    w = torch.randn(130, 256).bfloat16()
    qw, sb = fb.quantize_weight_block(w)
    assert sb.shape == (2, 2)
    assert (fb.dequantize_weight(qw, sb) - w.float()).abs().max() < 0.07 * w.float().abs().max()


def test_block_linear_cpu_forward_backward():
    torch.manual_seed(1)
    x = torch.randn(3, 4, 128).bfloat16().requires_grad_(True)
    w = (torch.randn(64, 128) * 0.1).bfloat16().requires_grad_(True)
    y = fb.fp8_block_linear(x, w)
    ref = x.float() @ w.float().t()
    assert (y.float() - ref).abs().max() < 0.06 * ref.abs().max() + 0.02
    y.float().sum().backward()
    assert x.grad.shape == x.shape and w.grad.shape == w.shape


@pytest.mark.gpu
@pytest.mark.parametrize("m,n,k,bias", [(128, 128, 128, False), (300, 200, 640, True), (4096, 2048, 4096, False), (17, 4096, 1024, True)])
def test_block_gemm_matches_dequantised_matmul(m, n, k, bias):
    from astrai_b200.ops import native

    native.require()
    g = torch.Generator(device="cuda").manual_seed(m + k)
    col_gain = torch.where(torch.arange(k, device="cuda") % 256 < 128, 1.0, 20.0)  # alternate quiet and loud K blocks
    x = (torch.randn(m, k, device="cuda", generator=g) * col_gain).bfloat16()
    w = (torch.randn(n, k, device="cuda", generator=g) * 0.05).bfloat16()
    bv = torch.randn(n, device="cuda", generator=g).bfloat16() if bias else None
    a_q, sa_t = fb.quantize_act_block(x)
    b_q, sb = fb.quantize_weight_block(w)
    # the kernels quantise like the PyTorch statement (scales exact, codes equal up to round-half cases)
    a_ref, sa_ref = fb.quantize_act_block_reference(x)
    b_ref, sb_ref = fb.quantize_weight_block_reference(w)
    assert torch.allclose(sa_t, sa_ref, rtol=1e-6) and torch.allclose(sb, sb_ref, rtol=1e-6)
    assert (a_q.float() - a_ref.float()).abs().max() <= 32 and (a_q.float() != a_ref.float()).float().mean() < 1e-3
    got = fb.mm_fp8_block(a_q, sa_t, b_q, sb, bv).float()
    ref = fb.dequantize_act(a_q, sa_t).double() @ fb.dequantize_weight(b_q, sb).double().t()
    if bias:
        ref = ref + bv.double()
    err = (got.double() - ref).abs().max().item()
    assert err <= 2 ** -7 * ref.abs().max().item() + 1e-4, err  # fp32 accumulation + bf16 rounding of the result
    full = x.float() @ w.float().t()
    assert (got - (full + (bv.float() if bias else 0))).abs().max().item() < 0.05 * full.abs().max().item()
    assert native.kernel_status(torch.device("cuda")) == 0


@pytest.mark.parametrize("backward", ["fp8", "bf16"])
def test_block_linear_gradients_track_bf16(backward):
    """All three products of the layer (forward, input gradient, weight gradient) on the block-scaled path against plain
    arithmetic on the same operands (CPU statement of the kernels)."""
    from astrai_b200.ops.fp8_block import fp8_block_linear

    torch.manual_seed(3)
    x = (torch.randn(2, 128, 256) * 0.5).requires_grad_(True)   # 256 tokens: a multiple of 128, so the weight gradient is quantised too
    w = torch.nn.Parameter(torch.randn(384, 256) * 0.05)
    b = torch.nn.Parameter(torch.randn(384) * 0.1)
    y = fp8_block_linear(x, w, b, backward=backward)
    ref = torch.nn.functional.linear(x, w, b)
    assert (y.float() - ref).abs().max() < 0.05 * ref.abs().max()
    gy = torch.randn_like(ref)
    y.float().backward(gy)
    gx, gw, gb = torch.autograd.grad(ref, (x, w, b), gy)
    tol = 0.06 if backward == "fp8" else 0.02
    assert (x.grad - gx).abs().max() < tol * gx.abs().max()
    assert (w.grad - gw).abs().max() < tol * gw.abs().max()
    assert torch.allclose(b.grad, gb, atol=0.05, rtol=0.02)


def test_block_backward_falls_back_for_ragged_token_counts_and_feeds_main_grad():
    from astrai_b200.ops.fp8_block import fp8_block_linear

    torch.manual_seed(4)
    x = torch.randn(100, 128, requires_grad=True)  # 100 tokens: the gradient products stay in bf16
    w = torch.nn.Parameter(torch.randn(128, 128) * 0.05)
    w.main_grad = torch.zeros(128, 128)
    y = fp8_block_linear(x, w)
    gy = torch.randn_like(y, dtype=torch.float32)
    y.float().backward(gy)
    assert w.grad is None and (w.main_grad - gy.t() @ x.detach()).abs().max() < 0.02 * (gy.t() @ x.detach()).abs().max()
    with pytest.raises(ValueError):
        fp8_block_linear(x, w, backward="int4")


def test_block_recipe_routes_linears_through_the_block_path():
    from astrai_b200 import ops
    from astrai_b200.ops import fp8

    torch.manual_seed(5)
    x, w = torch.randn(128, 256), torch.randn(128, 256) * 0.05
    plain = ops.linear(x, w)
    with fp8.fp8_autocast(recipe=fp8.BlockScaling()):
        block = ops.linear(x, w)
        narrow = ops.linear(torch.randn(16, 64), torch.randn(32, 64))  # 64 columns: per-tensor scaling instead
    assert block.dtype == torch.bfloat16 and narrow.shape == (16, 32)
    diff = (block.float() - plain).abs().max()
    assert 0 < diff < 0.05 * plain.abs().max()  # quantised, and close
    assert fp8.BlockScaling().measure_first and fp8.BlockScaling(backward="bf16").backward == "bf16"


@pytest.mark.gpu
@pytest.mark.parametrize("m,n,k", [(256, 384, 256), (1024, 2048, 512)])
def test_block_linear_backward_on_the_kernels_tracks_bf16(m, n, k):
    """Forward and both gradient products through the block GEMM on the GPU against fp32 arithmetic on the operands."""
    from astrai_b200.ops.fp8_block import fp8_block_linear

    torch.manual_seed(6)
    x = (torch.randn(m, k, device="cuda") * 0.5).bfloat16().requires_grad_(True)
    w = (torch.randn(n, k, device="cuda") * 0.05).bfloat16().requires_grad_(True)
    y = fp8_block_linear(x, w)
    gy = torch.randn(m, n, device="cuda").bfloat16()
    y.backward(gy)
    xf, wf, gf = x.detach().float(), w.detach().float(), gy.float()
    ref_y, ref_gx, ref_gw = xf @ wf.t(), gf @ wf, gf.t() @ xf
    for got, ref in ((y, ref_y), (x.grad, ref_gx), (w.grad, ref_gw)):
        assert (got.float() - ref).abs().max().item() < 0.06 * ref.abs().max().item()
