"""FP8 recipes, scaling state and autocast (CPU), and the tcgen05 fp8 kernels against explicit quantise -> fp32 matmul."""

import pytest
import torch

from astrai_b200.ops import fp8


def test_recipes_compute_scale_from_amax():
    d = fp8.DelayedScaling(history_len=4, margin=1)
    hist = torch.tensor([1.0, 8.0, 2.0, 4.0])
    assert d.scale_from_history(hist, "e4m3").item() == pytest.approx(8.0 / 448.0 / 2)
    assert fp8.DynamicScaling().scale_from_history(torch.tensor([3.0]), "e5m2").item() == pytest.approx(3.0 / 57344.0)
    assert fp8.FP8Format.HYBRID.fwd() == "e4m3" and fp8.FP8Format.HYBRID.bwd() == "e5m2" and fp8.FP8Format.E5M2.fwd() == "e5m2"


def test_meta_ring_is_delayed_max():
    meta = fp8.FP8TensorMeta("cpu", fp8.DelayedScaling(history_len=3))
    meta.seed("x", torch.tensor([2.0, -4.0]), "e4m3")
    assert meta.scale["x"].item() == pytest.approx(4.0 / 448.0)
    for a in (1.0, 1.0, 1.0):
        meta.update("x", torch.tensor(a), "e4m3")
    assert meta.scale["x"].item() == pytest.approx(1.0 / 448.0)  # the 4.0 fell out of the window


def test_autocast_routes_linear_and_restores_state():
    from astrai_b200 import ops

    torch.manual_seed(0)
    x = torch.randn(32, 64, requires_grad=True)
    w = torch.randn(48, 64, requires_grad=True)
    ref = x @ w.t()
    assert not fp8.autocast_state().enabled
    with ops.fp8_autocast(recipe=fp8.DynamicScaling()):
        assert fp8.autocast_state().enabled
        y = ops.linear(x, w)
    assert not fp8.autocast_state().enabled and hasattr(w, "_fp8_meta")
    assert (y.float() - ref).abs().max().item() < 0.08 * ref.abs().max().item()  # e4m3 has a 3-bit mantissa
    y.float().sum().backward()
    dx_ref = torch.ones(32, 48) @ w.detach()
    assert (x.grad - dx_ref).abs().max().item() < 0.1 * dx_ref.abs().max().item()
    assert w.grad is not None and w.grad.shape == w.shape


@pytest.mark.gpu
@pytest.mark.parametrize("fmt", ["e4m3", "e5m2"])
@pytest.mark.parametrize("rows,cols", [(256, 512), (130, 72), (64, 1032)])
def test_quantize_kernel_matches_torch_cast(fmt, rows, cols):
    torch.manual_seed(1)
    x = (torch.randn(rows, cols, device="cuda") * 3).bfloat16()
    scale = torch.tensor([0.02], device="cuda")
    q, qt, amax = fp8.quantize_bf16(x, scale, fmt, with_transpose=True)
    ref = (x.float() / 0.02).clamp(-fp8.FP8_MAX[fmt], fp8.FP8_MAX[fmt]).to(q.dtype)
    assert amax.item() == pytest.approx(x.float().abs().max().item())
    mism = (q.float() != ref.float()).float().mean().item()
    assert mism < 2e-3  # identical up to ties resolved on a bf16-rounded quotient
    assert (q.float() - ref.float()).abs().max().item() <= ref.float().abs().max().item() * 0.13
    assert torch.equal(qt.float(), q.float().t())


@pytest.mark.gpu
@pytest.mark.parametrize("m,n,k", [(256, 512, 256), (384, 272, 1040), (128, 256, 64)])
def test_fp8_gemm_matches_quantized_reference(m, n, k):
    torch.manual_seed(2)
    a = torch.randn(m, k, device="cuda").bfloat16()
    b = torch.randn(n, k, device="cuda").bfloat16()
    bias = torch.randn(n, device="cuda").bfloat16()
    sa = (a.float().abs().max() / 448.0).reshape(1)
    sb = (b.float().abs().max() / 57344.0).reshape(1)
    aq, _, _ = fp8.quantize_bf16(a, sa, "e4m3")
    bq, _, _ = fp8.quantize_bf16(b, sb, "e5m2")  # mixed formats in one MMA
    out = fp8.mm_fp8(aq, bq, sa, sb, bias)
    ref = (aq.float() @ bq.float().t()) * (sa * sb) + bias.float()
    assert torch.allclose(out.float(), ref, atol=0.125, rtol=0.01)
    from astrai_b200.ops import native

    assert native.kernel_status(a.device) == 0


@pytest.mark.gpu
def test_fp8_linear_autocast_trains_on_gpu():
    from astrai_b200 import ops

    torch.manual_seed(3)
    x = torch.randn(256, 512, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(384, 512, device="cuda") * 0.05).bfloat16().requires_grad_(True)
    with ops.fp8_autocast():
        y = ops.linear(x, w)
    ref = x.detach().float() @ w.detach().float().t()
    assert (y.float() - ref).abs().max().item() < 0.08 * ref.abs().max().item()
    g = torch.randn_like(y)
    y.backward(g)
    dx_ref, dw_ref = g.float() @ w.detach().float(), g.float().t() @ x.detach().float()
    assert (x.grad.float() - dx_ref).abs().max().item() < 0.12 * dx_ref.abs().max().item()
    assert (w.grad.float() - dw_ref).abs().max().item() < 0.12 * dw_ref.abs().max().item()
