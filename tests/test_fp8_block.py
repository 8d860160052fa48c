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
