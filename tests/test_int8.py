"""int8 quantisation and the W8A8 linear layer: CPU statements, and the kind::i8 GEMM against exact integer math."""

import pytest
import torch

from astrai_b200.ops import int8


def test_quantize_rows_reference_roundtrip():
    torch.manual_seed(0)
    x = torch.randn(5, 32)
    x[2] = 0
    q, s = int8.quantize_rows(x)
    assert q.dtype == torch.int8 and s.shape == (5,)
    assert s[2] == 1 and (q[2] == 0).all()
    assert (q.abs().amax(dim=1)[[0, 1, 3, 4]] == 127).all()
    assert ((q.float() * s[:, None]) - x).abs().max() <= s.max() * 0.5 + 1e-6


def test_int8_linear_module_cpu_matches_dequantised_matmul():
    torch.manual_seed(1)
    lin = torch.nn.Linear(32, 16, bias=True)
    q = int8.Int8Linear.from_linear(lin)
    x = torch.randn(4, 32).bfloat16()
    got = q(x).float()
    ref = lin(x.float())
    assert (got - ref).abs().max() < 0.05 * ref.abs().max() + 0.05
    sd = q.state_dict()
    assert set(sd) == {"weight_q", "weight_scale", "bias"}


def test_quantize_model_replaces_linears_but_not_the_head():
    m = torch.nn.ModuleDict({"body": torch.nn.Linear(32, 32, bias=False), "lm_head": torch.nn.Linear(32, 64, bias=False)})
    assert int8.quantize_model_int8(m) == 1
    assert isinstance(m["body"], int8.Int8Linear) and isinstance(m["lm_head"], torch.nn.Linear)


@pytest.mark.gpu
@pytest.mark.parametrize("m,n,k,bias", [(128, 256, 128, False), (300, 520, 1040, True), (5, 64, 64, False), (2048, 4096, 4096, True)])
def test_int8_gemm_matches_exact_integer_math(m, n, k, bias):
    from astrai_b200.ops import native

    native.require()
    g = torch.Generator(device="cuda").manual_seed(m + n)
    a = torch.randint(-127, 128, (m, k), device="cuda", generator=g, dtype=torch.int32).to(torch.int8)
    b = torch.randint(-127, 128, (n, k), device="cuda", generator=g, dtype=torch.int32).to(torch.int8)
    sa = torch.rand(m, device="cuda", generator=g) * 0.01 + 1e-3
    sb = torch.rand(n, device="cuda", generator=g) * 0.01 + 1e-3
    bv = torch.randn(n, device="cuda", generator=g).bfloat16() if bias else None
    got = int8.mm_int8(a, sa, b, sb, bv).float()
    acc = (a.double() @ b.double().t())  # exact: |acc| < 2^53
    ref = acc * sa.double()[:, None] * sb.double()[None, :]
    if bias:
        ref = ref + bv.double()
    err = (got.double() - ref).abs().max().item()
    assert err <= 2 ** -8 * ref.abs().max().item() + 1e-6, err  # bf16 rounding of the result only
    assert native.kernel_status(torch.device("cuda")) == 0


@pytest.mark.gpu
def test_int8_quantize_kernel_matches_reference_and_linear_is_close():
    from astrai_b200.ops import native

    native.require()
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn(257, 1024, device="cuda", generator=g).bfloat16()
    x[7] = 0
    q, s = int8.quantize_rows(x)
    qr, sr = int8.quantize_rows_reference(x)
    assert torch.allclose(s, sr, rtol=1e-6)
    assert (q.int() - qr.int()).abs().max().item() <= 1  # round-half cases may differ by one step
    w = (torch.randn(512, 1024, device="cuda", generator=g) * 0.05).bfloat16()
    lin = torch.nn.Linear(1024, 512, bias=False, device="cuda", dtype=torch.bfloat16)
    with torch.no_grad():
        lin.weight.copy_(w)
    y = int8.Int8Linear.from_linear(lin)(x).float()
    ref = x.float() @ w.float().t()
    assert (y - ref).abs().max().item() < 0.04 * ref.abs().max().item()
