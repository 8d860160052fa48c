"""Attention back ends as pluggable classes (selection by name, enum member, class, instance and environment), a back end
of one's own behind the models and the scheduler, and the functional attention calls under the reference's names."""

import math

import pytest
import torch

from helpers import tiny_config


@pytest.fixture(autouse=True)
def _clean_environment(monkeypatch):
    monkeypatch.delenv("ASTR_BACKEND", raising=False)
    monkeypatch.delenv("ASTRAI_B200_ATTN", raising=False)


def test_factory_lists_the_builtin_backends_under_the_references_names_too():
    from astrai_b200 import ops

    assert ops.AttentionBackendFactory.list_registered()[:4] == ["cuda", "flash", "tcgen05", "torch_native"]
    assert isinstance(ops.AttentionBackendFactory.create("cuda"), ops.Tcgen05Backend)
    assert ops.CudaBackend.supports_graph() and not ops.TorchNativeBackend.supports_graph()
    assert ops.TorchNativeBackend.supports() is True


@pytest.mark.parametrize("how", ["name", "enum", "class", "instance", "with_instance"])
def test_selection_forms_are_equivalent_and_unwind(how):
    from astrai_b200 import ops
    from astrai_b200.ops import backend as b

    native = ops.ATTN_BACKEND.TORCH_NATIVE
    assert b.get_backend("cuda", use_default=False) is None
    if how == "with_instance":
        with ops.TorchNativeBackend() as selected:
            assert isinstance(selected, ops.TorchNativeBackend) and b.get_backend("cuda") is native
    else:
        choice = {"name": "torch_native", "enum": native, "class": ops.TorchNativeBackend, "instance": ops.TorchNativeBackend()}[how]
        with ops.attn_backend(choice):
            assert b.get_backend("cuda") is native and b.get_backend("cuda", use_default=False) is native and b.explicit()
            with ops.attn_backend(ops.CudaBackend):
                assert b.get_backend("cuda") is ops.ATTN_BACKEND.TCGEN05
            assert b.get_backend("cuda") is native
    assert b.get_backend("cuda", use_default=False) is None and b.get_backend("cuda") is ops.ATTN_BACKEND.TCGEN05
    assert b.get_backend("cpu") is native


def test_unknown_names_and_objects_are_rejected():
    from astrai_b200 import ops

    for bad in ("metal", 3, object):
        with pytest.raises(ValueError):
            with ops.attn_backend(bad):
                pass


class _Counting:
    """Mixin of the test back ends below: the plain-PyTorch statement, counting what it is asked to do."""

    def __init__(self):
        self.calls = []

    def _math(self, q, k, v, kv_cache, layer_id, attn_mask, is_causal, fwd):
        from astrai_b200 import ops
        from astrai_b200.ops.attention import dense_attention
        from astrai_b200.ops.paged_attention import cached_attention

        self.calls.append((fwd, tuple(q.shape), layer_id))
        with ops.attn_backend("torch_native"):  # from inside: the built-in statement
            if fwd is None:
                return dense_attention(q, k, v, attn_mask, is_causal)
            return cached_attention(q, k, v, kv_cache, layer_id, attn_mask, is_causal, fwd)


def _own_backend_class():
    from astrai_b200 import ops

    class Own(_Counting, ops.AttentionBackend):
        def fwd_prefill(self, q, k, v, kv_cache, layer_id, attn_mask=None, is_causal=False):
            return self._math(q, k, v, kv_cache, layer_id, attn_mask, is_causal, None if kv_cache is None else "prefill")

        def fwd_decode(self, q, k, v, kv_cache, layer_id, attn_mask=None, is_causal=False):
            return self._math(q, k, v, kv_cache, layer_id, attn_mask, is_causal, "decode")

    return Own


def test_a_backend_of_ones_own_receives_the_models_attention_calls():
    from astrai_b200 import ops
    from astrai_b200.models import AutoRegressiveLM
    from astrai_b200.ops import backend as b

    torch.manual_seed(0)
    model = AutoRegressiveLM(tiny_config()).eval()
    ids = torch.randint(1, 1000, (2, 9))
    want = model(ids)["logits"]
    own = _own_backend_class()()
    with ops.attn_backend(own):
        assert b.get_backend("cuda") is own and b.current_custom() is own
        got = model(ids)["logits"]
    assert b.current_custom() is None
    assert torch.allclose(got, want, atol=1e-6)
    assert [c[2] for c in own.calls] == [0, 1] and all(c[0] is None and c[1][:2] == (2, 9) for c in own.calls)
    with own:  # an instance selects itself
        assert b.current_custom() is own
    with pytest.raises(NotImplementedError):
        with ops.attn_backend(ops.AttentionBackend()):  # the base class computes nothing
            model(ids)


def test_registered_backend_is_selectable_by_name_environment_and_scheduler(monkeypatch):
    from astrai_b200 import ops
    from astrai_b200.inference import InferenceScheduler
    from astrai_b200.models import AutoRegressiveLM
    from astrai_b200.ops import backend as b
    from astrai_b200.tokenize import AutoTokenizer  # noqa: F401 - the scheduler only needs encode / stop ids below

    Own = _own_backend_class()
    name = "own_for_tests"
    if name not in ops.AttentionBackendFactory.list_registered():
        ops.AttentionBackendFactory.register(name)(Own)
    with ops.attn_backend(name):
        assert isinstance(b.current_custom(), ops.AttentionBackend) and type(b.current_custom()).__name__ == "Own"
    monkeypatch.setenv("ASTR_BACKEND", name)
    first = b.get_backend("cuda")
    assert type(first).__name__ == "Own" and b.get_backend("cuda") is first  # built once per value of the variable
    with ops.attn_backend("torch_native"):
        assert b.get_backend("cuda") is first  # the environment wins over a context
    monkeypatch.delenv("ASTR_BACKEND")

    class Tok:
        stop_ids = [0]

        def encode(self, text):
            return [5, 6, 7]

    torch.manual_seed(0)
    model = AutoRegressiveLM(tiny_config(max_position_embeddings=64)).eval()
    plain = InferenceScheduler(model, Tok(), max_batch_size=2, max_seq_len=32, enable_cuda_graph=False).run_batch(
        [[30, 31, 32], [40, 41]], max_tokens=4, temperature=0.0)
    own = Own()
    sched = InferenceScheduler(model, Tok(), max_batch_size=2, max_seq_len=32, enable_cuda_graph=False, backend=own)
    assert sched.backend_name == "Own"
    with ops.attn_backend(own):  # the synchronous path runs on the caller's thread
        assert sched.run_batch([[30, 31, 32], [40, 41]], max_tokens=4, temperature=0.0) == plain
    kinds = {c[0] for c in own.calls}
    assert kinds == {"prefill", "decode"}


# ------------------------------------------------------------------------------------------------ functional calls
def _ref_attention(q, k, v, keep):
    """fp64 softmax attention, blhd, grouped-query heads, boolean ``keep`` broadcastable to [B, H, Lq, Lk]."""
    hq, hkv = q.shape[2], k.shape[2]
    qt, kt, vt = (t.double().transpose(1, 2) for t in (q, k, v))
    kt, vt = kt.repeat_interleave(hq // hkv, 1), vt.repeat_interleave(hq // hkv, 1)
    s = qt @ kt.transpose(-1, -2) / math.sqrt(q.shape[-1])
    s = s.masked_fill(~keep, float("-inf"))
    return (torch.softmax(s, -1) @ vt).transpose(1, 2).float()


def test_attn_prefill_aligns_causality_to_the_end_of_the_keys_and_takes_masks_and_layouts():
    from astrai_b200 import ops

    torch.manual_seed(1)
    q, k, v = torch.randn(2, 3, 4, 8), torch.randn(2, 7, 2, 8), torch.randn(2, 7, 2, 8)
    tri = torch.ones(3, 7, dtype=torch.bool).tril(diagonal=4)[None, None]
    assert torch.allclose(ops.attn_prefill(q, k, v, is_causal=True), _ref_attention(q, k, v, tri), atol=1e-5)
    everything = torch.ones(1, 1, 3, 7, dtype=torch.bool)
    assert torch.allclose(ops.attn_prefill(q, k, v), _ref_attention(q, k, v, everything), atol=1e-5)
    keys = torch.ones(2, 7, dtype=torch.bool)
    keys[0, :2] = False
    assert torch.allclose(ops.attn_prefill(q, k, v, mask=keys, is_causal=True), _ref_attention(q, k, v, tri & keys[:, None, None, :]), atol=1e-5)
    full = torch.rand(2, 3, 7) > 0.3
    full[..., 0] = True
    assert torch.allclose(ops.attn_prefill(q, k, v, mask=full), _ref_attention(q, k, v, full[:, None]), atol=1e-5)
    bhld = ops.attn_prefill(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True, layout=ops.TensorLayout.BHLD)
    assert bhld.shape == (2, 4, 3, 8) and torch.allclose(bhld.transpose(1, 2), _ref_attention(q, k, v, tri), atol=1e-5)
    square = torch.randn(2, 7, 4, 8)
    assert torch.allclose(ops.attn_prefill(square, k, v, is_causal=True),
                          _ref_attention(square, k, v, torch.ones(7, 7, dtype=torch.bool).tril()[None, None]), atol=1e-5)


def test_attn_decode_is_one_query_over_all_keys():
    from astrai_b200 import ops

    torch.manual_seed(2)
    q, k, v = torch.randn(3, 1, 4, 8), torch.randn(3, 5, 4, 8), torch.randn(3, 5, 4, 8)
    want = _ref_attention(q, k, v, torch.ones(1, 1, 1, 5, dtype=torch.bool))
    assert torch.allclose(ops.attn_decode(q, k, v, is_causal=True), want, atol=1e-5)
    with pytest.raises(ValueError):
        ops.attn_decode(torch.randn(3, 2, 4, 8), k, v)


def test_attn_paged_decode_reads_the_pool_through_the_slot_table_and_appends_the_new_token():
    from astrai_b200 import ops

    torch.manual_seed(3)
    hq, hkv, d, slots = 4, 2, 8, 40
    k_pool, v_pool = torch.randn(slots, hkv, d), torch.randn(slots, hkv, d)
    table = torch.zeros(3, 12, dtype=torch.int32)
    perm = torch.randperm(slots)
    table[0, :5], table[2, :9] = perm[:5].int(), perm[5:14].int()  # rows 0 and 2 are in use, lengths 5 and 9
    rows, indptr = torch.tensor([2, 0], dtype=torch.int32), torch.tensor([0, 9, 14], dtype=torch.int32)
    q = torch.randn(2, hq, d)
    new_k, new_v = torch.randn(2, hkv, d), torch.randn(2, hkv, d)
    k_before = k_pool.clone()
    out = ops.attn_paged_decode(q, k_pool, v_pool, table, rows, indptr, new_k=new_k, new_v=new_v)
    assert out.shape == (2, hq, d)
    last = torch.stack([table[2, 8], table[0, 4]]).long()
    assert torch.equal(k_pool[last], new_k) and torch.equal(v_pool[last], new_v)
    untouched = torch.ones(slots, dtype=torch.bool)
    untouched[last] = False
    assert torch.equal(k_pool[untouched], k_before[untouched])
    for i, (row, n) in enumerate(((2, 9), (0, 5))):
        idx = table[row, :n].long()
        want = _ref_attention(q[i][None, None], k_pool[idx][None], v_pool[idx][None], torch.ones(1, 1, 1, n, dtype=torch.bool))
        assert torch.allclose(out[i], want[0, 0], atol=1e-5)
    again = torch.empty_like(out)
    assert ops.attn_paged_decode(q, k_pool, v_pool, table, rows, indptr, out_buf=again) is again  # the pool holds the token already
    assert torch.allclose(again, out, atol=1e-6)


def test_rotary_helpers_under_the_references_names():
    from astrai_b200 import ops
    from astrai_b200.models import apply_rotary_emb, get_rotary_emb

    table = get_rotary_emb(8, 16, base=10000.0)
    assert table.shape == (16, 4, 2) and torch.allclose(table[0], torch.tensor([1.0, 0.0]).expand(4, 2))
    x = torch.randn(2, 16, 3, 8)
    y = apply_rotary_emb(x, table[None].expand(2, -1, -1, -1))
    assert y.shape == x.shape and torch.allclose(y[:, 0], x[:, 0], atol=1e-6)  # position 0 is not rotated
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1), atol=1e-5)  # a rotation
    assert torch.allclose(ops.apply_rotary_emb(x, table[None].expand(2, -1, -1, -1)), y)


def test_kernel_names_and_availability():
    from astrai_b200 import ops

    assert {"gemm", "flash_fwd", "flash_bwd", "paged_decode_append_", "sample_rows", "adamw_"} <= set(ops.KERNEL_NAMES)
    assert ops.is_available("no_such_kernel") is False
    assert isinstance(ops.is_available("gemm"), bool) and isinstance(ops.is_available(), bool)


def test_attn_paged_prefill_attends_from_the_last_positions_of_each_request():
    from astrai_b200 import ops

    torch.manual_seed(4)
    hq, hkv, d, slots = 4, 2, 8, 48
    k_pool, v_pool = torch.randn(slots, hkv, d), torch.randn(slots, hkv, d)
    table = torch.zeros(4, 16, dtype=torch.int32)
    perm = torch.randperm(slots).int()
    table[1, :10], table[3, :6] = perm[:10], perm[10:16]
    rows = torch.tensor([3, 1], dtype=torch.int32)
    kv_indptr, qo_indptr = torch.tensor([0, 6, 16], dtype=torch.int32), torch.tensor([0, 6, 9], dtype=torch.int32)  # 6 of 6, last 3 of 10
    q = torch.randn(9, hq, d)
    before = k_pool.clone()
    out = ops.attn_paged_prefill(q, k_pool, v_pool, table, rows, kv_indptr, qo_indptr)
    assert out.shape == (9, hq, d) and torch.equal(k_pool, before)  # the pool is read, not changed
    for i, (row, m, n, start) in enumerate(((3, 6, 6, 0), (1, 3, 10, 6))):
        idx = table[row, :n].long()
        keep = torch.ones(m, n, dtype=torch.bool).tril(diagonal=n - m)[None, None]
        want = _ref_attention(q[start:start + m][None], k_pool[idx][None], v_pool[idx][None], keep)[0]
        assert torch.allclose(out[start:start + m], want, atol=1e-5), i


def test_small_helpers_under_the_references_names():
    from astrai_b200 import ops
    from astrai_b200.data.dataset import validate_keys
    from astrai_b200.models.layers import ntk_base
    from astrai_b200.models.lm import process_attention_mask
    from astrai_b200.preprocessing.core import infer_dtype

    x = torch.arange(2 * 3 * 4.0).view(2, 3, 4)
    assert ops.repeat_kv(x, 1) is x and ops.repeat_kv(x, 2).shape == (2, 6, 4)
    assert torch.equal(ops.repeat_kv(x, 2)[:, 0], x[:, 0]) and torch.equal(ops.repeat_kv(x, 2)[:, 1], x[:, 0])
    assert isinstance(ops.flash_attn_available(), bool)
    assert ntk_base(10000.0, 64, 1.0) == 10000.0 and ntk_base(10000.0, 64, 4.0) == pytest.approx(10000.0 * 4 ** (64 / 62))
    m2, m3, m4 = torch.ones(2, 5), torch.ones(2, 5, 5), torch.ones(2, 1, 5, 5)
    assert process_attention_mask(None) is None and process_attention_mask(m2).shape == (2, 1, 1, 5)
    assert process_attention_mask(m3).shape == (2, 1, 5, 5) and process_attention_mask(m4) is m4
    assert infer_dtype([0.5]) is torch.float32 and infer_dtype([1, 2]) is torch.int32 and infer_dtype([]) is torch.int32

    class Has:
        keys = ["sequence", "loss_mask"]

    validate_keys(Has(), ["sequence"])
    validate_keys(Has(), [])
    with pytest.raises(KeyError, match="position_ids"):
        validate_keys(Has(), ["sequence", "position_ids"])
