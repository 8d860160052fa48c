"""SFT, DPO and GRPO steps on the GPU: their attention restrictions (packed documents, padding) run on the
variable-length tcgen05 flash kernels, and the loss equals the dense-boolean-mask statement in fp32."""

import copy

import pytest
import torch

pytestmark = pytest.mark.gpu


def _models():
    from astrai_b200.config import AutoRegressiveLMConfig
    from astrai_b200.models import AutoRegressiveLM

    cfg = AutoRegressiveLMConfig(vocab_size=512, hidden_size=256, num_hidden_layers=2, rms_norm_eps=1e-6, intermediate_size=512,
                                 tie_word_embeddings=False, max_position_embeddings=512, rope_theta=10000.0,
                                 num_attention_heads=2, num_key_value_heads=1)
    torch.manual_seed(5)
    native = AutoRegressiveLM(cfg).cuda().to(torch.bfloat16)
    oracle = copy.deepcopy(native).float()  # same (bf16-rounded) weights, fp32 math, library attention with dense masks
    return native, oracle


class _Spy:
    def __init__(self, monkeypatch):
        from astrai_b200.ops import flash

        self.calls = 0
        real = flash.flash_attention_varlen

        def spy(*a, **k):
            self.calls += 1
            return real(*a, **k)

        monkeypatch.setattr(flash, "flash_attention_varlen", spy)


def _dense_masks(monkeypatch):
    """Force the strategies back onto the reference's dense boolean masks (for the oracle pass)."""
    from astrai_b200.trainer import strategy as S

    monkeypatch.setattr(S, "doc_attention", lambda pos: S.make_doc_boundary_mask(pos.cuda()))
    monkeypatch.setattr(S, "padded_causal_attention", lambda valid: S.causal_padding_mask(valid.cuda()))


def test_sft_packed_documents_run_on_flash_varlen(monkeypatch):
    from astrai_b200.trainer.strategy import SFTStrategy

    native, oracle = _models()
    g = torch.Generator().manual_seed(0)
    b, s = 2, 384
    ids = torch.randint(1, 512, (b, s + 1), generator=g)
    pos = torch.cat([torch.arange(100), torch.arange(150), torch.arange(134)])[None].repeat(b, 1)
    pos[1] = torch.cat([torch.arange(384)])  # one row with a single document
    batch = {"input_ids": ids[:, :-1], "target_ids": ids[:, 1:], "position_ids": pos,
             "loss_mask": torch.rand(b, s, generator=g) > 0.3}
    spy = _Spy(monkeypatch)
    loss = SFTStrategy(native, "cuda")(batch)["loss"]
    loss.backward()
    assert spy.calls == 2  # one variable-length flash call per layer, no dense mask anywhere
    _dense_masks(monkeypatch)
    ref = SFTStrategy(oracle, "cuda")(batch)["loss"]
    assert abs(float(loss) - float(ref)) < 3e-2
    gnorm = torch.sqrt(sum(p.grad.float().pow(2).sum() for p in native.parameters() if p.grad is not None))
    assert torch.isfinite(gnorm) and float(gnorm) > 0


def test_dpo_and_grpo_padding_run_on_flash_varlen(monkeypatch):
    from astrai_b200.trainer.strategy import DPOStrategy, GRPOStrategy

    native, oracle = _models()
    ref_native, ref_oracle = copy.deepcopy(native).eval(), copy.deepcopy(oracle).eval()
    g = torch.Generator().manual_seed(1)
    n, s = 2, 257
    chosen = torch.randint(1, 512, (n, s), generator=g)
    rejected = torch.randint(1, 512, (n, s), generator=g)
    chosen[0, 200:] = 0      # right padding (token id 0)
    rejected[1, 130:] = 0
    cm, rm = (chosen != 0).float(), (rejected != 0).float()
    cm[:, :40] = 0
    rm[:, :40] = 0           # the prompt part carries no loss
    batch = {"chosen": chosen, "rejected": rejected, "chosen_mask": cm, "rejected_mask": rm}
    spy = _Spy(monkeypatch)
    loss = DPOStrategy(native, "cuda", ref_model=ref_native)(batch)["loss"]
    loss.backward()
    assert spy.calls == 4  # policy and frozen model, two layers each
    # GRPO: left-padded prompts followed by right-padded responses
    b, grp, plen, rlen = 2, 2, 128, 129
    prompts = torch.randint(1, 512, (b, plen), generator=g)
    prompts[0, :50] = 0
    responses = torch.randint(1, 512, (b, grp, rlen), generator=g)
    masks = torch.ones(b, grp, rlen)
    masks[1, 0, 90:] = 0
    responses[1, 0, 90:] = 0
    gbatch = {"prompts": prompts, "responses": responses, "masks": masks, "rewards": torch.tensor([[1.0, 0.0], [0.2, 0.9]])}
    spy.calls = 0
    gl = GRPOStrategy(native, "cuda", old_model=ref_native, ref_model=ref_native)(gbatch)["loss"]
    gl.backward()
    assert spy.calls == 6 and torch.isfinite(gl)
    _dense_masks(monkeypatch)
    ref = DPOStrategy(oracle, "cuda", ref_model=ref_oracle)(batch)["loss"]
    assert abs(float(loss) - float(ref)) < 5e-2
    gref = GRPOStrategy(oracle, "cuda", old_model=ref_oracle, ref_model=ref_oracle)(gbatch)["loss"]
    assert abs(float(gl) - float(gref)) < 5e-2


def test_padding_inside_a_row_falls_back_to_the_dense_mask():
    from astrai_b200.trainer.strategy import padded_causal_attention

    valid = torch.tensor([[1, 1, 0, 1, 1, 0]]).bool()
    out = padded_causal_attention(valid)
    assert isinstance(out, torch.Tensor) and out.shape == (1, 1, 6, 6)
