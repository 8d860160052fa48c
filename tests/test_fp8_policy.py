"""The fp8 training policy on the CPU reference path: formats, scaling recipes, the amax rings, quantise / matmul
fallbacks and the fp8 linear's forward and backward against bf16 arithmetic (behaviours the reference checks in
``tests/extension/test_fp8_mma.py``; the kernel-side comparisons are in ``tests/test_fp8.py``)."""

import pytest
import torch

from astrai_b200.ops import fp8


def test_formats_pick_e4m3_forward_and_e5m2_backward_in_hybrid_mode():
    assert fp8.FP8Format("hybrid") is fp8.FP8Format.HYBRID
    assert (fp8.FP8Format.HYBRID.fwd(), fp8.FP8Format.HYBRID.bwd()) == ("e4m3", "e5m2")
    assert (fp8.FP8Format.E4M3.fwd(), fp8.FP8Format.E4M3.bwd()) == ("e4m3", "e4m3")
    assert (fp8.FP8Format.E5M2.fwd(), fp8.FP8Format.E5M2.bwd()) == ("e5m2", "e5m2")
    assert fp8.FP8_MAX == {"e4m3": 448.0, "e5m2": 57344.0}
    with pytest.raises(ValueError):
        fp8.FP8Format("e3m4")


def test_scale_maps_the_largest_amax_of_the_history_onto_the_format_range():
    r = fp8.DelayedScaling(history_len=4)
    hist = torch.tensor([1.0, 8.0, 2.0, 0.5])
    assert float(r.scale_from_history(hist, "e4m3")) == pytest.approx(8.0 / 448.0)
    assert float(r.scale_from_history(hist, "e5m2")) == pytest.approx(8.0 / 57344.0)
    assert float(fp8.DelayedScaling(margin=2).scale_from_history(hist, "e4m3")) == pytest.approx(8.0 / 448.0 / 4)
    assert float(r.scale_from_history(torch.zeros(4), "e4m3")) > 0  # never a zero scale
    assert fp8.DynamicScaling().measure_first and not fp8.DelayedScaling().measure_first


def test_meta_rings_replace_the_oldest_entry_and_rescale():
    meta = fp8.FP8TensorMeta("cpu", fp8.DelayedScaling(history_len=3))
    assert not any(meta.seeded.values())
    meta.seed("x", torch.tensor([[-4.0, 2.0]]), "e4m3")
    assert meta.seeded["x"] and meta.hist["x"].tolist() == [4.0] * 3 and float(meta.scale["x"]) == pytest.approx(4.0 / 448.0)
    for amax in (1.0, 2.0, 3.0):
        meta.update("x", torch.tensor(amax), "e4m3")
    assert meta.hist["x"].tolist() == [1.0, 2.0, 3.0] and float(meta.scale["x"]) == pytest.approx(3.0 / 448.0)
    meta.update("x", torch.tensor(0.5), "e4m3")  # wraps around: the 1.0 is the oldest
    assert meta.hist["x"].tolist() == [0.5, 2.0, 3.0]
    assert meta.hist["w"].tolist() == [1.0] * 3 and meta.idx == {"w": 0, "x": 1, "g": 0}  # the rings are independent


@pytest.mark.parametrize("fmt", ["e4m3", "e5m2"])
def test_quantise_fallback_saturates_reports_amax_and_transposes(fmt):
    x = torch.tensor([[0.5, -1.0, 1000.0], [0.25, 2.0, -3.0]])
    scale = torch.tensor([1.0 / 64])
    q, qt, amax = fp8.quantize_bf16(x, scale, fmt, with_transpose=True)
    assert q.dtype == (torch.float8_e4m3fn if fmt == "e4m3" else torch.float8_e5m2) and q.shape == (2, 3) and qt.shape == (3, 2)
    assert float(amax) == 1000.0
    back = q.float() * scale
    assert back[0, 2] == pytest.approx(min(1000.0, fp8.FP8_MAX[fmt] / 64))  # clipped to the format's largest value, not inf
    assert torch.allclose(back[:, :2], x[:, :2], rtol=0.13 if fmt == "e5m2" else 0.07)
    assert torch.equal(qt.float(), q.float().t())
    assert fp8.quantize_bf16(x, scale, fmt)[1] is None


def test_matmul_fallback_applies_both_scales_and_the_bias():
    torch.manual_seed(0)
    a, b = torch.randn(8, 32), torch.randn(16, 32)
    sa, sb = torch.tensor([a.abs().max() / 448]), torch.tensor([b.abs().max() / 448])
    qa, qb = fp8.quantize_bf16(a, sa)[0], fp8.quantize_bf16(b, sb)[0]
    bias = torch.randn(16)
    out = fp8.mm_fp8(qa, qb, sa, sb, bias, out_dtype=torch.float32)
    exact = (qa.float() * sa) @ (qb.float() * sb).t() + bias
    assert torch.allclose(out, exact, atol=1e-4)
    assert (out - (a @ b.t() + bias)).abs().max() < 0.06 * (a @ b.t()).abs().max()  # fp8 operands, a few percent
    assert fp8.mm_fp8(qa, qb, sa, sb).dtype == torch.bfloat16


@pytest.mark.parametrize("recipe", [fp8.DelayedScaling(), fp8.DynamicScaling()])
def test_fp8_linear_forward_and_backward_track_the_bf16_layer(recipe):
    torch.manual_seed(1)
    x = torch.randn(4, 6, 32, requires_grad=True)
    w = torch.nn.Parameter(torch.randn(48, 32) * 0.2)
    b = torch.nn.Parameter(torch.randn(48) * 0.1)
    with fp8.fp8_autocast(recipe=recipe):
        y = fp8.fp8_linear(x, w, b)
    assert y.shape == (4, 6, 48)
    ref = torch.nn.functional.linear(x, w, b)
    assert (y.float() - ref).abs().max() < 0.08 * ref.abs().max()
    gy = torch.randn_like(ref)
    y.float().backward(gy)
    gx, gw, gb = torch.autograd.grad(ref, (x, w, b), gy)
    assert (x.grad - gx).abs().max() < 0.15 * gx.abs().max()   # E5M2 gradients: two mantissa bits
    assert (w.grad - gw).abs().max() < 0.15 * gw.abs().max()
    assert torch.allclose(b.grad, gb, atol=0.05, rtol=0.02)    # a plain sum of the (bf16) output gradient
    meta = w._fp8_meta
    assert all(meta.seeded.values()) and isinstance(meta.recipe, type(recipe))


def test_delayed_recipe_uses_last_steps_amax_and_dynamic_the_current_one():
    w = torch.nn.Parameter(torch.ones(16, 16) * 0.1)
    small, large = torch.ones(16, 16), torch.ones(16, 16) * 100
    with fp8.fp8_autocast(recipe=fp8.DelayedScaling(history_len=1)):
        fp8.fp8_linear(small, w)
        first = float(w._fp8_meta.scale["x"])
        fp8.fp8_linear(large, w)           # quantised with the scale of the step before ...
        assert float(w._fp8_meta.scale["x"]) == pytest.approx(100.0 / 448.0)  # ... and leaves its own amax for the next
    assert first == pytest.approx(1.0 / 448.0)
    w2 = torch.nn.Parameter(torch.ones(16, 16) * 0.1)
    with fp8.fp8_autocast(recipe=fp8.DynamicScaling()):
        fp8.fp8_linear(small, w2)
        y = fp8.fp8_linear(large, w2)
    assert float(w2._fp8_meta.scale["x"]) == pytest.approx(100.0 / 448.0)
    assert torch.allclose(y.float(), torch.full((16, 16), 160.0), rtol=0.05)  # measured first: no saturation


def test_autocast_state_nests_and_restores():
    assert not fp8.autocast_state().enabled
    with fp8.fp8_autocast(fp8_format=fp8.FP8Format.E4M3, update_interval=4, margin=1):
        st = fp8.autocast_state()
        assert st.enabled and st.fp8_format is fp8.FP8Format.E4M3 and st.update_interval == 4 and st.recipe.margin == 1
        with fp8.fp8_autocast(enabled=False):
            assert not fp8.autocast_state().enabled
        assert fp8.autocast_state().enabled
    assert not fp8.autocast_state().enabled


def test_a_new_recipe_type_gets_a_fresh_meta_and_the_same_type_keeps_it():
    w = torch.nn.Parameter(torch.randn(16, 16))
    a = fp8.meta_for(w, fp8.DelayedScaling())
    assert fp8.meta_for(w, fp8.DelayedScaling(margin=3)) is a
    assert fp8.meta_for(w, fp8.DynamicScaling()) is not a


def test_only_bf16_cuda_multiples_of_16_are_eligible():
    x, w = torch.randn(32, 32), torch.randn(32, 32)
    assert not fp8.eligible(x, w)  # CPU tensors stay on the regular path


def test_state_object_and_per_operand_spellings_of_the_reference():
    from astrai_b200.ops import fp8

    state = fp8.fp8_state()
    assert state.enabled is False and isinstance(state.recipe, fp8.DelayedScaling) and state.fp8_format is fp8.FP8Format.HYBRID
    w = torch.nn.Parameter(torch.randn(8, 8))
    with fp8.fp8_autocast(recipe=fp8.DynamicScaling(), fp8_format=fp8.FP8Format.E4M3):
        assert state.enabled is True and isinstance(state.recipe, fp8.DynamicScaling) and state.fp8_format.bwd() == "e4m3"
        meta = state.get_weight_meta(w)
        assert state.get_weight_meta(w) is meta  # kept on the weight
    assert state.enabled is False
    meta.init_w(w, "e4m3")
    assert meta.seeded["w"] and float(meta.w_scale) == pytest.approx(float(w.abs().max()) / 448.0, rel=1e-5)
    meta.update_x(torch.tensor(4.48), "e4m3")
    meta.update_g(torch.tensor(57.344), "e5m2")
    assert float(meta.x_scale) == pytest.approx(0.01, rel=1e-5) and float(meta.g_scale) == pytest.approx(0.001, rel=1e-5)
    meta.init_x(torch.full((3,), 2.0), "e4m3")
    meta.init_g(torch.full((3,), 2.0), "e5m2")
    meta.update_w(torch.tensor(448.0), "e4m3")
    assert float(meta.w_scale) == pytest.approx(1.0)
    state.reset(w)
    assert not hasattr(w, "_fp8_meta") and state.get_weight_meta(w) is not meta


def test_process_wide_switch_reaches_other_threads_and_yields_to_a_block():
    import threading

    from astrai_b200.ops import fp8

    assert fp8.fp8_linear_enabled() is False
    fp8.fp8_linear_enable(True)
    try:
        seen = []
        t = threading.Thread(target=lambda: seen.append((fp8.fp8_linear_enabled(), type(fp8.autocast_state().recipe).__name__)))
        t.start()
        t.join()
        assert seen == [(True, "DelayedScaling")] and fp8.fp8_linear_enabled() is True
        with fp8.fp8_autocast(enabled=False):
            assert fp8.fp8_linear_enabled() is False
        fp8.fp8_linear_enable(True, recipe=fp8.DynamicScaling())
        assert isinstance(fp8.fp8_state().recipe, fp8.DynamicScaling)
    finally:
        fp8.fp8_linear_enable(False, recipe=fp8.DelayedScaling())
    assert fp8.fp8_linear_enabled() is False
    assert fp8.fp8_quantize is fp8.quantize_bf16 and fp8.fp8_gemm is fp8.mm_fp8
